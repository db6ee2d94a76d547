// Library-level entry points: version and status strings.
#include "common.cuh"

extern "C" int xlstm_version(void) { return 100; }  // major*100 + minor

extern "C" const char *xlstm_strerror(int status) {
    switch (status) {
        case XLSTM_OK: return "ok";
        case XLSTM_ERR_INVALID: return "invalid argument (null pointer, bad size or forbidden aliasing)";
        case XLSTM_ERR_UNSUPPORTED: return "shape, stride, alignment or dtype not supported by the kernels";
        case XLSTM_ERR_CUDA: return "CUDA runtime call or kernel launch failed";
        case XLSTM_ERR_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
        case XLSTM_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        case XLSTM_ERR_STATIC_SCRATCH: return "problem needs more scratch than the built-in static block holds; use the workspace entry point";
        default: return "unknown status";
    }
}
