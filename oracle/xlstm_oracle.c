/*
 * CPU oracle for the xLSTM inference hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA kernels are compared against.  It is a
 * plain-C restatement of the reference's torch / numpy arithmetic, written
 * from the formulas, one function per reference function.  Nothing in the
 * shipped package may call it: only tests, the smoke check and the
 * cpu-baseline leg of the benchmark do.
 *
 * Parity status: pinned.  Every function here is checked against fixtures
 * produced by importing the reference's own Python classes on CPU (see
 * tests/golden/make_golden.py) and against the literal known-answer inputs
 * of the reference's tests (tests/test_mlx_torch_numerical_parity.py:8-73,
 * tests/parity/test_numerical_parity.py:105-108).
 *
 * Reference functions restated (paths inside the reference project):
 *   xo_softcap            xlstm_metal/torch_native/blocks/soft_cap/soft_cap_kernel.metal:13-14
 *                         tests/parity/canonical_reference.py:18-23
 *   xo_mlstm_recurrent    xlstm_metal/torch_native/blocks/mlstm/mlstm_chunkwise/mlstm_recurrent_kernel_cell.py:53-161
 *                         tests/parity/canonical_reference.py:59-111
 *   xo_mlstm_chunkwise    xlstm_metal/mlx_jit/blocks/mlstm/mlstm_chunkwise/mlstm_parallel_kernel_cell.py:132-249
 *                         (inter-chunk carry: .../forward/mlstm_chunkwise_recurrent_fw_C.py:20-333,
 *                          intra-chunk + combine: .../forward/mlstm_chunkwise_parallel_fw_Hintra.py:22-406)
 *   xo_slstm_scan         xlstm_metal/torch_native/blocks/slstm/slstm_layers/stepwise/slstm_stepwise_kernel_cell.py:47-97
 *                         applied once per timestep as slstm_neuron.py:132-143 does
 *   xo_slstm_recurrent    kernel_development/xlstm/implementations/pytorch/xlstm_pytorch_enhanced.py:428-461
 *                         (BlockLinear :207-229, init_hidden :407-413)
 *   xo_rmsnorm            tests/parity/canonical_reference.py:26-33
 *   xo_multihead_rmsnorm  xlstm_metal/torch_native/blocks/mlstm/multihead_norm/multihead_norm.py:43-64
 *
 * All tensors are dense row-major fp32.  Loops over (batch, head) are
 * OpenMP-parallel so the same code doubles as the timed CPU baseline.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- helpers ---------------------------------------------------------- */

/* round an fp32 value to the nearest bf16 (ties to even), return as fp32:
 * this is what a torch op with a bfloat16 result does to its fp32 math. */
static inline float bf16r(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return x; /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    u &= 0xffff0000u;
    float y;
    memcpy(&y, &u, 4);
    return y;
}

/* the reference's forget-gate log-sigmoid, literally -log(1 + exp(-f))
 * (mlstm_recurrent_kernel_cell.py:117) */
static inline float logsig_naive(float f) { return -logf(1.0f + expf(-f)); }

/* torch.nn.functional.logsigmoid (used by the sLSTM step cell, :83-86) */
static inline float logsig_stable(float f) {
    return fminf(f, 0.0f) - log1pf(expf(-fabsf(f)));
}

int xo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void xo_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ---- soft-cap ---------------------------------------------------------- */

void xo_softcap(const float *x, float *y, long n, float cap) {
    if (cap <= 0.0f) { /* softcap.py:27-28: cap <= 0 is the identity */
        if (y != x) memcpy(y, x, (size_t)n * sizeof(float));
        return;
    }
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; ++i) y[i] = cap * tanhf(x[i] / cap);
}

/* ---- RMSNorm (glue around the hot path; used by model-level parity) ---- */

void xo_rmsnorm(const float *x, const float *w, float *y, long rows, int d, float eps) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r) {
        const float *xr = x + r * d;
        float *yr = y + r * d;
        float ss = 0.f;
        for (int j = 0; j < d; ++j) ss += xr[j] * xr[j];
        float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (int j = 0; j < d; ++j) yr[j] = xr[j] * inv * (w ? w[j] : 1.0f);
    }
}

/* x: [rows, NH, DH]; w: flat [NH*DH]; rms = sqrt(mean(x^2) + eps) per head */
void xo_multihead_rmsnorm(const float *x, const float *w, float *y, long rows, int NH, int DH, float eps) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows * NH; ++r) {
        const float *xr = x + r * DH;
        float *yr = y + r * DH;
        int head = (int)(r % NH);
        float ss = 0.f;
        for (int j = 0; j < DH; ++j) ss += xr[j] * xr[j];
        float rms = sqrtf(ss / (float)DH + eps);
        for (int j = 0; j < DH; ++j) yr[j] = (xr[j] / rms) * (w ? w[head * DH + j] : 1.0f);
    }
}

/*
 * mLSTM output epilogue (mlstm_output_cell.py:84-94 with multihead_norm.py:43-64):
 * h: [B,NH,S,dv]  og (output-gate pre-activation), y: [B,S,NH*dv]  w: flat [NH*dv] or NULL
 *   y[b,s,head*dv+j] = h[b,head,s,j] / sqrt(mean_j h^2 + eps) * w[head*dv+j] * sigmoid(og[b,s,head*dv+j])
 */
void xo_mlstm_output_gate(const float *h, const float *og, const float *w, float *y, int B, int NH, int S, int dv,
                          float eps) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)B * S * NH; ++r) {
        int head = (int)(r % NH);
        long bs = r / NH, b = bs / S, s = bs % S;
        const float *hr = h + ((b * NH + head) * S + s) * dv;
        const float *ogr = og + r * dv;
        float *yr = y + r * dv;
        float ss = 0.f;
        for (int j = 0; j < dv; ++j) ss += hr[j] * hr[j];
        float rms = sqrtf(ss / (float)dv + eps);
        for (int j = 0; j < dv; ++j)
            yr[j] = (hr[j] / rms) * (w ? w[head * dv + j] : 1.0f) * (1.0f / (1.0f + expf(-ogr[j])));
    }
}

/* y[m,n] = sum_k x[m,k] W[n,k] + bias[n]: nn.Linear as the reference's cells call it
 * (mlstm_projection_cell.py:85-96, mlstm_output_cell.py:84-99, mlstm_block.py:198-204) */
void xo_linear(const float *x, const float *W, const float *bias, float *y, long M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M * N; ++i) {
        long m = i / N;
        int n = (int)(i % N);
        double acc = 0.0;
        for (int k = 0; k < K; ++k) acc += (double)x[m * K + k] * (double)W[(long)n * K + k];
        y[i] = (float)acc + (bias ? bias[n] : 0.0f);
    }
}

/* SwiGLU gate, mlstm_block.py:198-204: y = silu(g) * u */
void xo_swiglu(const float *g, const float *u, float *y, long n) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; ++i) y[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
}

/*
 * Causal depthwise conv over tokens, channels last (depthwise_kernel.metal:12-44 for the layout;
 * tap order of the nn.Conv1d path, causal_conv1d.py:61-67: tap K-1 meets the current token):
 *   y[b,s,c] = act(bias[c] + sum_j w[c,j] * x[b, s-(K-1)+j, c]);  tokens < 0 from state [B,K-1,C] or zero.
 * state_out (or NULL): the last K-1 inputs of [state ; x].  act: 0 none, 1 SiLU (slstm_projection_cell.py:110-117).
 */
void xo_causal_conv1d(const float *x, const float *w, const float *bias, const float *state, float *state_out,
                      float *y, int B, int S, int C, int K, int act) {
    int H = K - 1;
    for (int b = 0; b < B; ++b) {
        for (int s = 0; s < S; ++s)
            for (int c = 0; c < C; ++c) {
                float acc = bias ? bias[c] : 0.0f;
                for (int j = 0; j < K; ++j) {
                    int t = s - H + j;
                    float xv = t >= 0 ? x[((long)b * S + t) * C + c]
                                      : (state ? state[((long)b * H + (H + t)) * C + c] : 0.0f);
                    acc += w[(long)c * K + j] * xv;
                }
                y[((long)b * S + s) * C + c] = act ? acc / (1.0f + expf(-acc)) : acc;
            }
        if (state_out)
            for (int j = 0; j < H; ++j)
                for (int c = 0; c < C; ++c) {
                    int t = S - H + j;
                    state_out[((long)b * H + j) * C + c] =
                        t >= 0 ? x[((long)b * S + t) * C + c] : (state ? state[((long)b * H + (H + t)) * C + c] : 0.0f);
                }
    }
}

/* ---- mLSTM recurrent sequence (the torch_native semantics of record) --- */
/*
 * q,k: [B,NH,S,dqk]  v: [B,NH,S,dv]  ig,fg: [B,NH,S]
 * C0: [B,NH,dqk,dv] n0: [B,NH,dqk] m0: [B,NH]   (all three NULL => zeros, m=0)
 * h: [B,NH,S,dv]; C1,n1,m1 like the inputs.
 * emulate_bf16 != 0 reproduces the cast points of the reference run with
 * compute_dtype=bfloat16, state_dtype=float32 (inputs must already hold
 * bf16-representable values): every torch op whose result dtype is bf16 is
 * rounded, fp32 state arithmetic is left alone.
 */
void xo_mlstm_recurrent(const float *q, const float *k, const float *v,
                        const float *ig, const float *fg,
                        const float *C0, const float *n0, const float *m0,
                        float *h, float *C1, float *n1, float *m1,
                        int B, int NH, int S, int dqk, int dv, float eps, int emulate_bf16) {
    const int BH = B * NH;
#pragma omp parallel for schedule(dynamic, 1)
    for (int bh = 0; bh < BH; ++bh) {
        float *C = C1 + (size_t)bh * dqk * dv;
        float *n = n1 + (size_t)bh * dqk;
        float m;
        if (C0) {
            memcpy(C, C0 + (size_t)bh * dqk * dv, sizeof(float) * dqk * dv);
            memcpy(n, n0 + (size_t)bh * dqk, sizeof(float) * dqk);
            m = m0[bh];
        } else {
            memset(C, 0, sizeof(float) * dqk * dv);
            memset(n, 0, sizeof(float) * dqk);
            m = 0.f;
        }
        float *qs = (float *)malloc(sizeof(float) * dqk);
        float *acc = (float *)malloc(sizeof(float) * dv);
        const float scale = emulate_bf16 ? bf16r(1.0f / sqrtf(bf16r((float)dqk))) : 1.0f / sqrtf((float)dqk);
        for (int t = 0; t < S; ++t) {
            const float *qt = q + ((size_t)bh * S + t) * dqk;
            const float *kt = k + ((size_t)bh * S + t) * dqk;
            const float *vt = v + ((size_t)bh * S + t) * dv;
            const float it = ig[(size_t)bh * S + t];
            const float ft = fg[(size_t)bh * S + t];
            float flog;
            if (emulate_bf16) { /* :117 with every intermediate a bf16 tensor */
                float e = bf16r(expf(-ft));
                float s = bf16r(1.0f + e);
                flog = -bf16r(logf(s));
            } else {
                flog = logsig_naive(ft);
            }
            /* :118-122 (bf16 + fp32 state promotes to fp32, so no rounding) */
            const float mnew = fmaxf(flog + m, it);
            const float fgate = expf(flog + m - mnew);
            const float igate = expf(it - mnew);
            /* :126-134 */
            for (int j = 0; j < dqk; ++j) {
                float *Cj = C + (size_t)j * dv;
                const float kj = kt[j];
                if (emulate_bf16) {
                    for (int c = 0; c < dv; ++c) Cj[c] = fgate * Cj[c] + igate * bf16r(kj * vt[c]);
                } else {
                    for (int c = 0; c < dv; ++c) Cj[c] = fgate * Cj[c] + igate * (kj * vt[c]);
                }
                n[j] = fgate * n[j] + igate * kj;
            }
            m = mnew;
            /* :140-152 */
            float qn = 0.f;
            for (int c = 0; c < dv; ++c) acc[c] = 0.f;
            if (emulate_bf16) {
                for (int j = 0; j < dqk; ++j) {
                    qs[j] = bf16r(qt[j] * scale);
                    qn += bf16r(bf16r(n[j]) * qs[j]);
                    const float *Cj = C + (size_t)j * dv;
                    for (int c = 0; c < dv; ++c) acc[c] += bf16r(bf16r(Cj[c]) * qs[j]);
                }
                qn = bf16r(qn);
                float maxval = bf16r(expf(-bf16r(m)));
                float den = bf16r(fmaxf(fabsf(qn), maxval) + bf16r(eps));
                float *ht = h + ((size_t)bh * S + t) * dv;
                for (int c = 0; c < dv; ++c) ht[c] = bf16r(bf16r(acc[c]) / den);
            } else {
                for (int j = 0; j < dqk; ++j) {
                    qs[j] = qt[j] * scale;
                    qn += n[j] * qs[j];
                    const float *Cj = C + (size_t)j * dv;
                    for (int c = 0; c < dv; ++c) acc[c] += Cj[c] * qs[j];
                }
                float den = fmaxf(fabsf(qn), expf(-m)) + eps;
                float *ht = h + ((size_t)bh * S + t) * dv;
                for (int c = 0; c < dv; ++c) ht[c] = acc[c] / den;
            }
        }
        m1[bh] = m;
        free(qs);
        free(acc);
    }
}

/* ---- mLSTM chunkwise (two-phase form; algebraically equal to the above) - */
/*
 * Same tensors as xo_mlstm_recurrent; S must be a multiple of L (the
 * reference neuron only ever hands whole chunks to the chunkwise cell,
 * mlx_jit/.../mlstm_neuron.py:225-243).  Per chunk with carried (C,n,m):
 *   b_t = cumsum logsig(f),  G = b_{L-1},  a_t = G - b_t + i_t
 *   m'  = max(G + m, max_t a_t)
 *   C'  = e^{G+m-m'} C + sum_t e^{a_t-m'} k_t (x) v_t ;  n' likewise
 *   m_t = max(b_t + m, max_{s<=t} (b_t - b_s + i_s))
 *   h_t = [e^{b_t+m-m_t} q~C + sum_{s<=t} e^{b_t-b_s+i_s-m_t} (q~.k_s) v_s] /
 *         (max(|same with n / 1|, e^{-m_t}) + eps)
 * No lower clamp on m_t: the torch_native recurrent cell has none.
 */
void xo_mlstm_chunkwise(const float *q, const float *k, const float *v,
                        const float *ig, const float *fg,
                        const float *C0, const float *n0, const float *m0,
                        float *h, float *C1, float *n1, float *m1,
                        int B, int NH, int S, int dqk, int dv, int L, float eps) {
    const int BH = B * NH;
    const int NC = S / L;
    const float scale = 1.0f / sqrtf((float)dqk);
#pragma omp parallel for schedule(dynamic, 1)
    for (int bh = 0; bh < BH; ++bh) {
        float *C = C1 + (size_t)bh * dqk * dv;
        float *n = n1 + (size_t)bh * dqk;
        float m;
        if (C0) {
            memcpy(C, C0 + (size_t)bh * dqk * dv, sizeof(float) * dqk * dv);
            memcpy(n, n0 + (size_t)bh * dqk, sizeof(float) * dqk);
            m = m0[bh];
        } else {
            memset(C, 0, sizeof(float) * dqk * dv);
            memset(n, 0, sizeof(float) * dqk);
            m = 0.f;
        }
        float *b = (float *)malloc(sizeof(float) * L);
        float *num = (float *)malloc(sizeof(float) * dv);
        float *w = (float *)malloc(sizeof(float) * L);
        for (int c = 0; c < NC; ++c) {
            const size_t t0 = (size_t)bh * S + (size_t)c * L;
            const float *ic = ig + t0, *fc = fg + t0;
            float run = 0.f;
            for (int t = 0; t < L; ++t) { run += logsig_naive(fc[t]); b[t] = run; }
            const float G = b[L - 1];
            /* outputs of this chunk, using the state before the chunk */
            for (int t = 0; t < L; ++t) {
                const float *qt = q + (t0 + t) * dqk;
                float mt = b[t] + m;
                for (int s = 0; s <= t; ++s) mt = fmaxf(mt, b[t] - b[s] + ic[s]);
                const float winter = expf(b[t] + m - mt);
                float den = 0.f;
                for (int cc = 0; cc < dv; ++cc) num[cc] = 0.f;
                float qn = 0.f;
                for (int j = 0; j < dqk; ++j) {
                    const float qj = qt[j] * scale;
                    qn += qj * n[j];
                    const float *Cj = C + (size_t)j * dv;
                    for (int cc = 0; cc < dv; ++cc) num[cc] += qj * Cj[cc];
                }
                for (int cc = 0; cc < dv; ++cc) num[cc] *= winter;
                den = winter * qn;
                for (int s = 0; s <= t; ++s) {
                    const float *ks = k + (t0 + s) * dqk;
                    const float *vs = v + (t0 + s) * dv;
                    float dot = 0.f;
                    for (int j = 0; j < dqk; ++j) dot += qt[j] * ks[j];
                    const float p = dot * scale * expf(b[t] - b[s] + ic[s] - mt);
                    den += p;
                    for (int cc = 0; cc < dv; ++cc) num[cc] += p * vs[cc];
                }
                const float d = fmaxf(fabsf(den), expf(-mt)) + eps;
                float *ht = h + (t0 + t) * dv;
                for (int cc = 0; cc < dv; ++cc) ht[cc] = num[cc] / d;
            }
            /* carry the state across the chunk */
            float mnew = G + m;
            for (int t = 0; t < L; ++t) mnew = fmaxf(mnew, G - b[t] + ic[t]);
            const float decay = expf(G + m - mnew);
            for (int t = 0; t < L; ++t) w[t] = expf(G - b[t] + ic[t] - mnew);
            for (int j = 0; j < dqk; ++j) {
                float *Cj = C + (size_t)j * dv;
                float nj = decay * n[j];
                for (int cc = 0; cc < dv; ++cc) Cj[cc] *= decay;
                for (int t = 0; t < L; ++t) {
                    const float kw = w[t] * k[(t0 + t) * dqk + j];
                    const float *vt = v + (t0 + t) * dv;
                    nj += kw;
                    for (int cc = 0; cc < dv; ++cc) Cj[cc] += kw * vt[cc];
                }
                n[j] = nj;
            }
            m = mnew;
        }
        m1[bh] = m;
        free(b);
        free(num);
        free(w);
    }
}

/* ---- sLSTM, packaged variant: scalar gates per head, state (c,n,m) ------ */
/*
 * z: [B,S,NH,H]  ig,fg,og: [B,S,NH] (already soft-capped)
 * c0,n0: [B,NH,H]  m0: [B,NH]  (all NULL => zeros)
 * h: [B,S,NH,H]; c1,n1,m1 final state.  One kernel-cell step per t.
 */
void xo_slstm_scan(const float *z, const float *ig, const float *fg, const float *og,
                   const float *c0, const float *n0, const float *m0,
                   float *h, float *c1, float *n1, float *m1,
                   int B, int S, int NH, int H, float eps) {
#pragma omp parallel for schedule(static)
    for (int bh = 0; bh < B * NH; ++bh) {
        const int bb = bh / NH, hd = bh % NH;
        float *c = c1 + (size_t)bh * H;
        float *n = n1 + (size_t)bh * H;
        float m = 0.f;
        if (c0) {
            memcpy(c, c0 + (size_t)bh * H, sizeof(float) * H);
            memcpy(n, n0 + (size_t)bh * H, sizeof(float) * H);
            m = m0[bh];
        } else {
            memset(c, 0, sizeof(float) * H);
            memset(n, 0, sizeof(float) * H);
        }
        for (int t = 0; t < S; ++t) {
            const size_t g = ((size_t)bb * S + t) * NH + hd;
            const float lf = logsig_stable(fg[g]);
            const float mnew = fmaxf(m + lf, ig[g]);
            const float igate = expf(ig[g] - mnew);
            const float fgate = expf(m + lf - mnew);
            const float ogate = 1.0f / (1.0f + expf(-og[g]));
            const float *zt = z + g * H;
            float *ht = h + g * H;
            for (int j = 0; j < H; ++j) {
                c[j] = fgate * c[j] + igate * tanhf(zt[j]);
                n[j] = fgate * n[j] + igate;
                ht[j] = ogate * c[j] / (fabsf(n[j]) + eps);
            }
            m = mnew;
        }
        m1[bh] = m;
    }
}

/* ---- sLSTM, block-diagonal recurrent variant: state (c,n,h,m) per unit -- */
/*
 * gx: [B,S,4,D] input-side pre-activations W_g x + b_g, gate order i,f,z,o
 *     (D = NH*dh).  R: [4,NH,dh,dh] with R[g][head][out][in] (nn.Linear
 *     layout), rb: [4,D] recurrent biases.  State c,n,h,m: [B,D]; NULL c0 =>
 *     init_hidden: c=h=m=0, n=1.  cap > 0 soft-caps the i and f
 *     pre-activations.  hs: [B,S,D] hidden outputs; final state in *1.
 */
void xo_slstm_recurrent(const float *gx, const float *R, const float *rb,
                        const float *c0, const float *n0, const float *h0, const float *m0,
                        float *hs, float *c1, float *n1, float *h1, float *m1,
                        int B, int S, int NH, int dh, float cap) {
    const int D = NH * dh;
#pragma omp parallel for schedule(static)
    for (int bh = 0; bh < B * NH; ++bh) {
        const int bb = bh / NH, hd = bh % NH;
        const size_t so = (size_t)bb * D + (size_t)hd * dh;
        float *c = c1 + so, *n = n1 + so, *hh = h1 + so, *m = m1 + so;
        float *hprev = (float *)malloc(sizeof(float) * dh);
        for (int j = 0; j < dh; ++j) {
            c[j] = c0 ? c0[so + j] : 0.f;
            n[j] = c0 ? n0[so + j] : 1.f;
            hh[j] = c0 ? h0[so + j] : 0.f;
            m[j] = c0 ? m0[so + j] : 0.f;
        }
        for (int t = 0; t < S; ++t) {
            memcpy(hprev, hh, sizeof(float) * dh);
            const float *gxt = gx + ((size_t)bb * S + t) * 4 * D;
            for (int j = 0; j < dh; ++j) {
                float pre[4];
                for (int g = 0; g < 4; ++g) {
                    const float *Rrow = R + (((size_t)g * NH + hd) * dh + j) * dh;
                    float acc = 0.f;
                    for (int kk = 0; kk < dh; ++kk) acc += Rrow[kk] * hprev[kk];
                    pre[g] = gxt[(size_t)g * D + hd * dh + j] + (acc + rb[(size_t)g * D + hd * dh + j]);
                }
                float it = pre[0], ft = pre[1];
                if (cap > 0.f) { it = cap * tanhf(it / cap); ft = cap * tanhf(ft / cap); }
                const float zt = tanhf(pre[2]);
                const float ot = 1.0f / (1.0f + expf(-pre[3]));
                const float mt = fmaxf(ft + m[j], it);
                const float ie = expf(it - mt);
                const float fe = expf(ft - mt + m[j]);
                c[j] = fe * c[j] + ie * zt;
                n[j] = fe * n[j] + ie;
                m[j] = mt;
                hh[j] = ot * (c[j] / fmaxf(n[j], 1.0f));
                hs[((size_t)bb * S + t) * D + hd * dh + j] = hh[j];
            }
        }
        free(hprev);
    }
}
