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
// one or a single decoded token.  A column is held by R lanes of a warp, each with DK/R consecutive
// rows in registers for the whole walk; sums over key channels are a fixed tree of adds and shuffles,
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
constexpr int NR = ((DK + R - 1) / R + 3) / 4 * 4;   // rows of the column each of them holds (a multiple of 4)
// A lane's rows are consecutive (row i belongs to lane i / NR) and lie NRP floats from the next
// lane's in shared memory: NRP = 4 mod 8, so the 16-byte loads of the lanes of a group fall into
// different banks.  Rows beyond DK are staged as zeros and need no guard.
constexpr int NRP = NR % 8 == 4 ? NR : NR + 4;
constexpr int ROWLEN = R * NRP;
constexpr int THREADS = 128;
constexpr int COLS = THREADS / R;               // value channels per CTA
constexpr int TC = DK > 256 ? 4 : 8;            // tokens staged per round

__device__ __forceinline__ int row_at(int i) { return (i / NR) * NRP + (i % NR); }

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
    __shared__ __align__(16) float qs[TC][ROWLEN], ks[TC][ROWLEN], as[TC][ROWLEN];
    __shared__ float vs[TC][COLS];
    const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
    const int tid = threadIdx.x, col = tid / R, rg = tid % R;
    const int t_begin = cu_q[b], t_end = cu_q[b + 1];
    const int slot = state_slots[b];
    const bool col_ok = c0 + col < dv;
    float* sp = state + (((size_t)slot * H + h) * DK) * dv + c0 + col;
    float S[NR];
#pragma unroll
    for (int n = 0; n < NR; ++n) {
        const int i = rg * NR + n;
        S[n] = (col_ok && i < DK) ? sp[(size_t)i * dv] : 0.f;
    }
    for (int e = tid; e < TC * ROWLEN; e += THREADS)       // rows beyond DK and the gaps stay zero
        (&qs[0][0])[e] = (&ks[0][0])[e] = (&as[0][0])[e] = 0.f;
    for (int t0 = t_begin; t0 < t_end; t0 += TC) {
        const int nt = min(TC, t_end - t0);
        __syncthreads();
        for (int e = tid; e < nt * DK; e += THREADS) {
            const int tok = e / DK, i = e - tok * DK;
            const size_t t = (size_t)(t0 + tok);
            const int at = row_at(i);
            qs[tok][at] = ld(q, t * q_stride + (size_t)h * DK + i) * q_scale;
            ks[tok][at] = ld(k, t * k_stride + (size_t)h * DK + i);
            float zz = z[t * z_stride + (size_t)h * DK + i];
            if (z_bias) zz += to_f32<TW>(z_bias[(size_t)h * DK + i]);
            as[tok][at] = expf(log_sigmoid_f(zz) * inv_tau);
        }
        for (int e = tid; e < nt * COLS; e += THREADS) {
            const int tok = e / COLS, c = e - tok * COLS;
            vs[tok][c] = c0 + c < dv ? ld(v, (size_t)(t0 + tok) * v_stride + (size_t)h * dv + c0 + c) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int tok = 0; tok < TC; ++tok) {
            if (tok < nt) {
                const float vj = vs[tok][col];
                const float4* a4 = reinterpret_cast<const float4*>(&as[tok][rg * NRP]);
                const float4* k4 = reinterpret_cast<const float4*>(&ks[tok][rg * NRP]);
                const float4* q4 = reinterpret_cast<const float4*>(&qs[tok][rg * NRP]);
                float o0 = 0.f, o1 = 0.f;
#pragma unroll
                for (int m = 0; m < NR / 4; ++m) {
                    const float4 a = a4[m], kk = k4[m], qq = q4[m];
                    S[4 * m + 0] = fmaf(a.x, S[4 * m + 0], kk.x * vj);
                    S[4 * m + 1] = fmaf(a.y, S[4 * m + 1], kk.y * vj);
                    S[4 * m + 2] = fmaf(a.z, S[4 * m + 2], kk.z * vj);
                    S[4 * m + 3] = fmaf(a.w, S[4 * m + 3], kk.w * vj);
                    o0 = fmaf(S[4 * m + 0], qq.x, o0);
                    o1 = fmaf(S[4 * m + 1], qq.y, o1);
                    o0 = fmaf(S[4 * m + 2], qq.z, o0);
                    o1 = fmaf(S[4 * m + 3], qq.w, o1);
                }
                const float o = group_sum(o0 + o1);
                if (rg == 0 && col_ok) out[((size_t)(t0 + tok) * H + h) * dv + c0 + col] = o;
            }
        }
    }
    if (col_ok) {
#pragma unroll
        for (int n = 0; n < NR; ++n) {
            const int i = rg * NR + n;
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
    __shared__ __align__(16) float rs[TC][ROWLEN], ks[TC][ROWLEN], ws[TC][ROWLEN], us[TC][ROWLEN], aus[TC][ROWLEN];
    __shared__ float vs[TC][COLS];
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
        const int i = rg * NR + n;
        S[n] = (col_ok && i < DK) ? sp[(size_t)i * dv] : 0.f;
    }
    for (int e = tid; e < TC * ROWLEN; e += THREADS)       // rows beyond DK and the gaps stay zero
        (&rs[0][0])[e] = (&ks[0][0])[e] = (&ws[0][0])[e] = (&us[0][0])[e] = (&aus[0][0])[e] = 0.f;
    for (int t0 = t_begin; t0 < t_end; t0 += TC) {
        const int nt = min(TC, t_end - t0);
        __syncthreads();
        for (int e = tid; e < nt * DK; e += THREADS) {
            const int tok = e / DK, i = e - tok * DK;
            const size_t t = (size_t)(t0 + tok);
            const size_t c = (size_t)h * DK + i;
            const int at = row_at(i);
            rs[tok][at] = ld(r, t * r_stride + c);
            ks[tok][at] = ld(k, t * k_stride + c);
            float zz = zw[t * zw_stride + c];
            if (zw_bias) zz += to_f32<TW>(zw_bias[c]);
            ws[tok][at] = expf(-decay_rate * sigmoid_f(zz));
            float az = ld(za, t * za_stride + c);
            if (za_bias) az += to_f32<TW>(za_bias[c]);
            aus[tok][at] = sigmoid_f(az);                     // times the unit key below
        }
        for (int e = tid; e < nt * COLS; e += THREADS) {
            const int tok = e / COLS, c = e - tok * COLS;
            vs[tok][c] = c0 + c < dv ? ld(v, (size_t)(t0 + tok) * v_stride + (size_t)h * dv + c0 + c) : 0.f;
        }
        __syncthreads();
        for (int tok = warp; tok < nt; tok += THREADS / 32) {  // unit keys: a warp a token
            float ss = 0.f;
            for (int i = lane; i < DK; i += 32) {
                const float x = ks[tok][row_at(i)];
                ss = fmaf(x, x, ss);
            }
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss + unit_eps);
            for (int i = lane; i < DK; i += 32) {
                const int at = row_at(i);
                const float u = ks[tok][at] * inv;
                us[tok][at] = u;
                aus[tok][at] *= u;
            }
        }
        __syncthreads();
#pragma unroll
        for (int tok = 0; tok < TC; ++tok) {
            if (tok < nt) {
                const float vj = vs[tok][col];
                const float4* u4 = reinterpret_cast<const float4*>(&us[tok][rg * NRP]);
                float d0 = 0.f, d1 = 0.f;
#pragma unroll
                for (int m = 0; m < NR / 4; ++m) {
                    const float4 u = u4[m];
                    d0 = fmaf(u.x, S[4 * m + 0], d0);
                    d1 = fmaf(u.y, S[4 * m + 1], d1);
                    d0 = fmaf(u.z, S[4 * m + 2], d0);
                    d1 = fmaf(u.w, S[4 * m + 3], d1);
                }
                const float dot = group_sum(d0 + d1);
                const float4* w4 = reinterpret_cast<const float4*>(&ws[tok][rg * NRP]);
                const float4* au4 = reinterpret_cast<const float4*>(&aus[tok][rg * NRP]);
                const float4* k4 = reinterpret_cast<const float4*>(&ks[tok][rg * NRP]);
                const float4* r4 = reinterpret_cast<const float4*>(&rs[tok][rg * NRP]);
                float o0 = 0.f, o1 = 0.f;
#pragma unroll
                for (int m = 0; m < NR / 4; ++m) {
                    const float4 w = w4[m], au = au4[m], kk = k4[m], rr = r4[m];
                    S[4 * m + 0] = fmaf(w.x, S[4 * m + 0], fmaf(-au.x, dot, kk.x * vj));
                    S[4 * m + 1] = fmaf(w.y, S[4 * m + 1], fmaf(-au.y, dot, kk.y * vj));
                    S[4 * m + 2] = fmaf(w.z, S[4 * m + 2], fmaf(-au.z, dot, kk.z * vj));
                    S[4 * m + 3] = fmaf(w.w, S[4 * m + 3], fmaf(-au.w, dot, kk.w * vj));
                    o0 = fmaf(S[4 * m + 0], rr.x, o0);
                    o1 = fmaf(S[4 * m + 1], rr.y, o1);
                    o0 = fmaf(S[4 * m + 2], rr.z, o0);
                    o1 = fmaf(S[4 * m + 3], rr.w, o1);
                }
                const float o = group_sum(o0 + o1);
                if (rg == 0 && col_ok) out[((size_t)(t0 + tok) * H + h) * dv + c0 + col] = o;
            }
        }
    }
    if (col_ok) {
#pragma unroll
        for (int n = 0; n < NR; ++n) {
            const int i = rg * NR + n;
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
