// Linear-attention recurrences over a per-request state matrix S [key channel][value channel]
// kept in fp32 (compiled for one key size RI_KDIM; any value size):
//
//   gated      S_t = diag(alpha_t) S_{t-1} + k_t v_t^T                          o_t = S_t^T q_t
//              alpha = sigmoid(z)^(1/tau), formed as exp(log_sigmoid(z) / tau)
//   delta      S_t = diag(w_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T   o_t = S_t^T r_t
//              u = k / sqrt(|k|^2 + unit_eps), w = exp(-decay_rate * sigmoid(z_w)), a = sigmoid(z_a)
//
// The columns of S do not mix, so a CTA owns a tile of value channels of one head of one batch
// entry and walks the entry's tokens in order, whatever their number: a prompt, a portion of
// one or a single decoded token.  A column is held by R lanes of a warp, each with DK/R of its
// rows in registers for the whole walk; sums over key channels are a fixed tree of shuffles,
// so a token's result has the same bits however the tokens were cut into steps or batches.
// Per round of TC tokens the CTA stages the vectors every column needs (decays, gates, unit
// keys: each formed once, in fp32) in shared memory.  Projections arrive in the activation
// dtype; the state, the decays and every sum are fp32.
#include "common.cuh"

#ifndef RI_KDIM
#error "compile with -DRI_KDIM=<key size>"
#endif

namespace {
constexpr int DK = RI_KDIM;
static_assert(DK >= 1 && DK <= 512, "key size up to 512");
constexpr int R = DK <= 64 ? 4 : 8;             // lanes that share a column
constexpr int NR = (DK + R - 1) / R;            // rows of the column each of them holds
constexpr int THREADS = 128;
constexpr int COLS = THREADS / R;               // value channels per CTA
constexpr int TC = DK > 256 ? 4 : 8;            // tokens staged per round

__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = 1; o < R; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T>
__device__ __forceinline__ float ld(const T* p, size_t i) { return to_f32<T>(p[i]); }

// q, k: [T, >= H*DK] with row strides; v: [T, >= H*dv]; z: fp32 logits of the decay [T, H*DK]
// (+ z_bias [H*DK] when given); out: fp32 [T, H*dv]; state: [slots][H][DK][dv] fp32.
template <typename TA, typename TW>
__global__ void __launch_bounds__(THREADS)
gated_scan_kernel(const TA* __restrict__ q, int q_stride, const TA* __restrict__ k, int k_stride,
                  const TA* __restrict__ v, int v_stride, const float* __restrict__ z, int z_stride,
                  const TW* __restrict__ z_bias, float q_scale, float inv_tau, float* __restrict__ out,
                  float* __restrict__ state, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                  int H, int dv) {
    pdl_trigger();
    pdl_wait();
    __shared__ float qs[TC][DK], ks[TC][DK], as[TC][DK], vs[TC][COLS];
    const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
    const int tid = threadIdx.x, col = tid / R, rg = tid % R;
    const int t_begin = cu_q[b], t_end = cu_q[b + 1];
    const int slot = state_slots[b];
    const bool col_ok = c0 + col < dv;
    float* sp = state + (((size_t)slot * H + h) * DK) * dv + c0 + col;
    float S[NR];
#pragma unroll
    for (int n = 0; n < NR; ++n) {
        const int i = rg + R * n;
        S[n] = (col_ok && i < DK) ? sp[(size_t)i * dv] : 0.f;
    }
    for (int t0 = t_begin; t0 < t_end; t0 += TC) {
        const int nt = min(TC, t_end - t0);
        __syncthreads();
        for (int e = tid; e < nt * DK; e += THREADS) {
            const int tok = e / DK, i = e - tok * DK;
            const size_t t = (size_t)(t0 + tok);
            qs[tok][i] = ld(q, t * q_stride + (size_t)h * DK + i) * q_scale;
            ks[tok][i] = ld(k, t * k_stride + (size_t)h * DK + i);
            float zz = z[t * z_stride + (size_t)h * DK + i];
            if (z_bias) zz += to_f32<TW>(z_bias[(size_t)h * DK + i]);
            as[tok][i] = expf(log_sigmoid_f(zz) * inv_tau);
        }
        for (int e = tid; e < nt * COLS; e += THREADS) {
            const int tok = e / COLS, c = e - tok * COLS;
            vs[tok][c] = c0 + c < dv ? ld(v, (size_t)(t0 + tok) * v_stride + (size_t)h * dv + c0 + c) : 0.f;
        }
        __syncthreads();
        for (int tok = 0; tok < nt; ++tok) {
            const float vj = vs[tok][col];
            float o = 0.f;
#pragma unroll
            for (int n = 0; n < NR; ++n) {
                const int i = rg + R * n;
                if (DK % R == 0 || i < DK) {
                    S[n] = fmaf(as[tok][i], S[n], ks[tok][i] * vj);
                    o = fmaf(S[n], qs[tok][i], o);
                }
            }
            o = group_sum(o);
            if (rg == 0 && col_ok) out[((size_t)(t0 + tok) * H + h) * dv + c0 + col] = o;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int n = 0; n < NR; ++n) {
            const int i = rg + R * n;
            if (i < DK) sp[(size_t)i * dv] = S[n];
        }
    }
}

// r, k, za: [T, >= H*DK]; v: [T, >= H*dv]; zw: fp32 logits of the decay [T, H*DK]; biases [H*DK] or null.
template <typename TA, typename TW>
__global__ void __launch_bounds__(THREADS)
delta_scan_kernel(const TA* __restrict__ r, int r_stride, const TA* __restrict__ k, int k_stride,
                  const TA* __restrict__ v, int v_stride, const TA* __restrict__ za, int za_stride,
                  const TW* __restrict__ za_bias, const float* __restrict__ zw, int zw_stride,
                  const TW* __restrict__ zw_bias, float decay_rate, float unit_eps, float* __restrict__ out,
                  float* __restrict__ state, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                  int H, int dv) {
    pdl_trigger();
    pdl_wait();
    __shared__ float rs[TC][DK], ks[TC][DK], ws[TC][DK], us[TC][DK], aus[TC][DK], vs[TC][COLS];
    const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
    const int tid = threadIdx.x, col = tid / R, rg = tid % R;
    const int lane = tid & 31, warp = tid >> 5;
    const int t_begin = cu_q[b], t_end = cu_q[b + 1];
    const int slot = state_slots[b];
    const bool col_ok = c0 + col < dv;
    float* sp = state + (((size_t)slot * H + h) * DK) * dv + c0 + col;
    float S[NR];
#pragma unroll
    for (int n = 0; n < NR; ++n) {
        const int i = rg + R * n;
        S[n] = (col_ok && i < DK) ? sp[(size_t)i * dv] : 0.f;
    }
    for (int t0 = t_begin; t0 < t_end; t0 += TC) {
        const int nt = min(TC, t_end - t0);
        __syncthreads();
        for (int e = tid; e < nt * DK; e += THREADS) {
            const int tok = e / DK, i = e - tok * DK;
            const size_t t = (size_t)(t0 + tok);
            const size_t c = (size_t)h * DK + i;
            rs[tok][i] = ld(r, t * r_stride + c);
            ks[tok][i] = ld(k, t * k_stride + c);
            float zz = zw[t * zw_stride + c];
            if (zw_bias) zz += to_f32<TW>(zw_bias[c]);
            ws[tok][i] = expf(-decay_rate * sigmoid_f(zz));
            float az = ld(za, t * za_stride + c);
            if (za_bias) az += to_f32<TW>(za_bias[c]);
            aus[tok][i] = sigmoid_f(az);                      // times the unit key below
        }
        for (int e = tid; e < nt * COLS; e += THREADS) {
            const int tok = e / COLS, c = e - tok * COLS;
            vs[tok][c] = c0 + c < dv ? ld(v, (size_t)(t0 + tok) * v_stride + (size_t)h * dv + c0 + c) : 0.f;
        }
        __syncthreads();
        for (int tok = warp; tok < nt; tok += THREADS / 32) {  // unit keys: a warp a token
            float ss = 0.f;
            for (int i = lane; i < DK; i += 32) ss = fmaf(ks[tok][i], ks[tok][i], ss);
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss + unit_eps);
            for (int i = lane; i < DK; i += 32) {
                const float u = ks[tok][i] * inv;
                us[tok][i] = u;
                aus[tok][i] *= u;
            }
        }
        __syncthreads();
        for (int tok = 0; tok < nt; ++tok) {
            const float vj = vs[tok][col];
            float dot = 0.f;
#pragma unroll
            for (int n = 0; n < NR; ++n) {
                const int i = rg + R * n;
                if (DK % R == 0 || i < DK) dot = fmaf(us[tok][i], S[n], dot);
            }
            dot = group_sum(dot);
            float o = 0.f;
#pragma unroll
            for (int n = 0; n < NR; ++n) {
                const int i = rg + R * n;
                if (DK % R == 0 || i < DK) {
                    S[n] = fmaf(ws[tok][i], S[n], fmaf(-aus[tok][i], dot, ks[tok][i] * vj));
                    o = fmaf(S[n], rs[tok][i], o);
                }
            }
            o = group_sum(o);
            if (rg == 0 && col_ok) out[((size_t)(t0 + tok) * H + h) * dv + c0 + col] = o;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int n = 0; n < NR; ++n) {
            const int i = rg + R * n;
            if (i < DK) sp[(size_t)i * dv] = S[n];
        }
    }
}
}  // namespace

RI_API int ri_recurrent_key_dim() { return DK; }

RI_API int ri_gated_scan(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride,
                         const float* z, int z_stride, const void* z_bias, int act_dtype, int w_dtype,
                         float q_scale, float inv_tau, float* out, float* state, const int* cu_q,
                         const int* state_slots, int entries, int H, int dv, void* stream) {
    if (entries <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((dv + COLS - 1) / COLS, H, entries);
#define RI_GS(TA, TW) RI_CHECKED(ri_launch(gated_scan_kernel<TA, TW>, grid, dim3(THREADS), 0, s, (const TA*)q, q_stride, \
        (const TA*)k, k_stride, (const TA*)v, v_stride, z, z_stride, (const TW*)z_bias, q_scale, inv_tau, out, state, \
        cu_q, state_slots, H, dv))
    if (act_dtype == RI_BF16 && w_dtype == RI_BF16) RI_GS(bf16, bf16);
    else if (act_dtype == RI_BF16) RI_GS(bf16, float);
    else if (w_dtype == RI_BF16) RI_GS(float, bf16);
    else RI_GS(float, float);
#undef RI_GS
    return ri_launch_status();
}

RI_API int ri_delta_scan(const void* r, int r_stride, const void* k, int k_stride, const void* v, int v_stride,
                         const void* za, int za_stride, const void* za_bias, const float* zw, int zw_stride,
                         const void* zw_bias, int act_dtype, int w_dtype, float decay_rate, float unit_eps,
                         float* out, float* state, const int* cu_q, const int* state_slots, int entries, int H,
                         int dv, void* stream) {
    if (entries <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((dv + COLS - 1) / COLS, H, entries);
#define RI_DS(TA, TW) RI_CHECKED(ri_launch(delta_scan_kernel<TA, TW>, grid, dim3(THREADS), 0, s, (const TA*)r, r_stride, \
        (const TA*)k, k_stride, (const TA*)v, v_stride, (const TA*)za, za_stride, (const TW*)za_bias, zw, zw_stride, \
        (const TW*)zw_bias, decay_rate, unit_eps, out, state, cu_q, state_slots, H, dv))
    if (act_dtype == RI_BF16 && w_dtype == RI_BF16) RI_DS(bf16, bf16);
    else if (act_dtype == RI_BF16) RI_DS(bf16, float);
    else if (w_dtype == RI_BF16) RI_DS(float, bf16);
    else RI_DS(float, float);
#undef RI_DS
    return ri_launch_status();
}

RI_API void ri_set_pdl(int on) { ri_pdl_flag() = on ? 1 : 0; }
