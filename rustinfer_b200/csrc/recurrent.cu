// Linear-attention recurrences over a per-request state matrix S [key channel][value channel]
// kept in fp32 (compiled for one key size RI_KDIM; any value size):
//
//   gated      S_t = diag(alpha_t) S_{t-1} + k_t v_t^T                          o_t = S_t^T q_t
//   delta      S_t = diag(w_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T   o_t = S_t^T r_t
//
// The decays alpha and w, the unit keys u and the products a * u arrive as fp32 vectors per token
// (made from the projections by kernels that run over all tokens at once, sequence_parts.cu).
//
// The columns of S do not mix, so a CTA owns a tile of value channels of one head of one batch
// entry and walks the entry's tokens in order, whatever their number: a prompt, a portion of
// one or a single decoded token.  Four warps compute.  A lane holds NR consecutive rows of C
// columns in registers for the whole walk, R lanes of a warp share those columns: a row's decay,
// key and query come from shared memory once and serve C columns (one column a lane made the walk
// wait for shared memory: a 16-byte load a multiply-add).  Sums over key channels are a fixed tree
// of adds and shuffles, taken for four tokens together so that the shuffles overlap; a token's
// result has the same bits however the tokens were cut into steps or batches.  Four more warps
// load: while a round of TC tokens is computed they fetch the next round's vectors (all loads of a
// round in flight at once, four elements each) and lay them into the other half of shared memory.
// Projections arrive in the activation dtype; the state, the decays and every sum are fp32.
//
// The state of one (slot, head) is stored value channel by value channel, [dv][DKP] with
// DKP = R * NR >= DK rows (the rows beyond DK stay zero), so that a lane's rows are 16-byte
// vectors and a warp reads and writes whole lines.
#include "common.cuh"

#ifndef RI_KDIM
#error "compile with -DRI_KDIM=<key size>"
#endif

namespace {
constexpr int DK = RI_KDIM;
static_assert(DK >= 1 && DK <= 512, "key size up to 512");
// Lanes that share a column: as few as leave a lane at most 4 rows, up to a whole warp.
constexpr int R = DK <= 16 ? 4 : DK <= 32 ? 8 : DK <= 64 ? 16 : 32;
constexpr int NR = ((DK + R - 1) / R + 3) / 4 * 4;   // rows of a column each of them holds (a multiple of 4)
constexpr int DKP = R * NR;                     // rows of a stored column
constexpr int C = NR <= 8 ? 4 : 2;              // columns a lane holds
// A lane's rows are consecutive (row i belongs to lane i / NR) and lie NRP floats from the next
// lane's in shared memory: NRP = 4 mod 8, so the 16-byte loads of eight lanes fall into
// different banks.  Rows beyond DK are zeros there and need no guard.
constexpr int NRP = NR % 8 == 4 ? NR : NR + 4;
constexpr int ROWLEN = R * NRP;
constexpr int WORKERS = 128;                    // threads that compute; as many load
constexpr int THREADS = 2 * WORKERS;
constexpr int COLS = WORKERS / R * C;           // value channels per CTA
constexpr int TC = DK <= 128 ? 16 : DK <= 256 ? 8 : 4;    // tokens per round
constexpr int TB = 4;                           // tokens whose sums over key channels are taken together
constexpr int PER = (TC * DK + WORKERS - 1) / WORKERS;    // elements of a vector a loading thread stages per round
constexpr int PER4 = (TC * DK / 4 + WORKERS - 1) / WORKERS;   // the same in groups of four

constexpr int half_floats(int arrays) { return arrays * TC * ROWLEN + TC * COLS; }

__device__ __forceinline__ int row_at(int i) { return (i / NR) * NRP + (i % NR); }

__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = R / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sums of N values over the R lanes of a group with fewer shuffles than N butterflies: at every
// offset (R/2 down to 1) a lane hands half of its values to its partner and keeps the sums of the
// other half, until one value is left, which the remaining offsets sum as a butterfly.  Every value
// goes through the same offsets in the same order as in group_sum, so its sum has the same bits.
// On return the lane holds the sums of the values first .. first + count - 1 in x[0 .. count - 1];
// lanes for which `owner` is false hold copies.
template <int N>
struct GroupSums {
    float x[N];
    int first, count;
    bool owner;
    __device__ __forceinline__ void run(int rg) {
        first = 0;
        owner = true;
        reduce<N, R / 2>(rg);
    }
    template <int n, int o>
    __device__ __forceinline__ void reduce(int rg) {
        if constexpr (o == 0) {
            count = n;
        } else if constexpr (n > 1) {
            const bool upper = (rg & o) != 0;
#pragma unroll
            for (int i = 0; i < n / 2; ++i) {
                const float send = upper ? x[i] : x[i + n / 2];
                const float keep = upper ? x[i + n / 2] : x[i];
                x[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
            }
            if (upper) first += n / 2;
            reduce<n / 2, o / 2>(rg);
        } else {
            x[0] += __shfl_xor_sync(0xffffffffu, x[0], o);
            if (rg & o) owner = false;
            reduce<1, o / 2>(rg);
        }
    }
};

// The sums of C values over the lanes of a group, every sum on every lane: scattered sums as above,
// then the lanes hand them back over the same offsets in reverse (9 shuffles for 4 values over a warp
// where 4 butterflies take 20).
__device__ __forceinline__ void all_sums(float (&d)[C], int rg) {
    GroupSums<C> g;
#pragma unroll
    for (int j = 0; j < C; ++j) g.x[j] = d[j];
    g.run(rg);
    d[0] = g.x[0];
    int have = 1;
#pragma unroll
    for (int half = 1; half < C; half *= 2) {                // the last halving offset first
        const int o = (R / 2) / (C / (2 * half));
        const bool upper = (rg & o) != 0;
#pragma unroll
        for (int i = 0; i < C / 2; ++i) {
            if (i < have) {
                const float got = __shfl_xor_sync(0xffffffffu, d[i], o);
                const float own = d[i];
                d[i] = upper ? got : own;
                d[i + have] = upper ? own : got;
            }
        }
        have *= 2;
    }
}

template <typename T>
__device__ __forceinline__ float ld(const T* p, size_t i) { return to_f32<T>(p[i]); }

// four consecutive elements from an address that is a multiple of four elements
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ float4 scaled(float4 v, float s) { return make_float4(v.x * s, v.y * s, v.z * s, v.w * s); }

// the lane's rows of its C columns: column j of the tile at sp + j * DKP
__device__ __forceinline__ void load_state(float (&S)[C][NR], const float* sp, const bool (&ok)[C]) {
#pragma unroll
    for (int j = 0; j < C; ++j)
#pragma unroll
        for (int m = 0; m < NR / 4; ++m) {
            const float4 x = ok[j] ? reinterpret_cast<const float4*>(sp + (size_t)j * DKP)[m] : make_float4(0.f, 0.f, 0.f, 0.f);
            S[j][4 * m] = x.x; S[j][4 * m + 1] = x.y; S[j][4 * m + 2] = x.z; S[j][4 * m + 3] = x.w;
        }
}
__device__ __forceinline__ void store_state(const float (&S)[C][NR], float* sp, const bool (&ok)[C]) {
#pragma unroll
    for (int j = 0; j < C; ++j)
        if (ok[j]) {
#pragma unroll
            for (int m = 0; m < NR / 4; ++m)
                reinterpret_cast<float4*>(sp + (size_t)j * DKP)[m] =
                    make_float4(S[j][4 * m], S[j][4 * m + 1], S[j][4 * m + 2], S[j][4 * m + 3]);
        }
}

// The round's values of the CTA's columns: loaded with the round's other vectors (addresses clamped to
// the tile, as theirs are), stored after them, so that a round costs the loaders one trip to memory.
constexpr int PERV = (TC * COLS + WORKERS - 1) / WORKERS;
template <typename TA>
__device__ __forceinline__ void load_values(float (&vv)[PERV], const TA* v, int v_stride, int t0, int nt, int h, int dv,
                                            int c0, int lt) {
#pragma unroll
    for (int j = 0; j < PERV; ++j) {
        const int e = min(lt + j * WORKERS, nt * COLS - 1);
        const int tok = e / COLS, c = min(e - tok * COLS, dv - 1 - c0);
        vv[j] = ld(v, (size_t)(t0 + tok) * v_stride + (size_t)h * dv + c0 + c);
    }
}
__device__ __forceinline__ void store_values(float* vs, const float (&vv)[PERV], int nt, int dv, int c0, int lt) {
#pragma unroll
    for (int j = 0; j < PERV; ++j) {
        const int e = lt + j * WORKERS;
        if (e < nt * COLS) {
            const int tok = e / COLS, c = e - tok * COLS;
            vs[tok * COLS + c] = c0 + c < dv ? vv[j] : 0.f;
        }
    }
}

// One token of one column from four rows' vectors: the arithmetic every kernel of this file shares.
//   gated:  S <- a S + k v;                      o += S q
//   delta:  S <- w S + (-au dot + k v);          o += S r      (dot: the old state's u^T S, summed before)
__device__ __forceinline__ void gated_rows(float* S, const float4& a, const float4& k, const float4& q, float vj,
                                           float& o0, float& o1) {
    S[0] = fmaf(a.x, S[0], k.x * vj);
    S[1] = fmaf(a.y, S[1], k.y * vj);
    S[2] = fmaf(a.z, S[2], k.z * vj);
    S[3] = fmaf(a.w, S[3], k.w * vj);
    o0 = fmaf(S[0], q.x, o0);
    o1 = fmaf(S[1], q.y, o1);
    o0 = fmaf(S[2], q.z, o0);
    o1 = fmaf(S[3], q.w, o1);
}
__device__ __forceinline__ void dot_rows(const float* S, const float4& u, float& d0, float& d1) {
    d0 = fmaf(u.x, S[0], d0);
    d1 = fmaf(u.y, S[1], d1);
    d0 = fmaf(u.z, S[2], d0);
    d1 = fmaf(u.w, S[3], d1);
}
__device__ __forceinline__ void delta_rows(float* S, const float4& w, const float4& au, const float4& k, const float4& r,
                                           float dot, float vj, float& o0, float& o1) {
    S[0] = fmaf(w.x, S[0], fmaf(-au.x, dot, k.x * vj));
    S[1] = fmaf(w.y, S[1], fmaf(-au.y, dot, k.y * vj));
    S[2] = fmaf(w.z, S[2], fmaf(-au.z, dot, k.z * vj));
    S[3] = fmaf(w.w, S[3], fmaf(-au.w, dot, k.w * vj));
    o0 = fmaf(S[0], r.x, o0);
    o1 = fmaf(S[1], r.y, o1);
    o0 = fmaf(S[2], r.z, o0);
    o1 = fmaf(S[3], r.w, o1);
}

// ------------------------------------------------------------------------------- gated
struct GatedHalf {
    float *q, *k, *a, *v;
    __device__ GatedHalf(float* base) : q(base), k(base + TC * ROWLEN), a(base + 2 * TC * ROWLEN), v(base + 3 * TC * ROWLEN) {}
};

// One token for this lane's rows of its C columns: the state update and, per column, the lane's part
// of the output's sum over key channels (group_sum adds the parts of a group's lanes).
__device__ __forceinline__ void gated_token(float (&S)[C][NR], const GatedHalf& b, int tok, int rg, int cg, float (&part)[C]) {
    const float4* a4 = reinterpret_cast<const float4*>(b.a + tok * ROWLEN + rg * NRP);
    const float4* k4 = reinterpret_cast<const float4*>(b.k + tok * ROWLEN + rg * NRP);
    const float4* q4 = reinterpret_cast<const float4*>(b.q + tok * ROWLEN + rg * NRP);
    float vj[C], o0[C], o1[C];
#pragma unroll
    for (int j = 0; j < C; ++j) {
        vj[j] = b.v[tok * COLS + cg * C + j];
        o0[j] = o1[j] = 0.f;
    }
#pragma unroll
    for (int m = 0; m < NR / 4; ++m) {
        const float4 a = a4[m], kk = k4[m], qq = q4[m];
#pragma unroll
        for (int j = 0; j < C; ++j) gated_rows(&S[j][4 * m], a, kk, qq, vj[j], o0[j], o1[j]);
    }
#pragma unroll
    for (int j = 0; j < C; ++j) part[j] = o0[j] + o1[j];
}

// q, k: [T, >= H*DK] with row strides; v: [T, >= H*dv]; alpha: fp32 decays [T, H*DK];
// out: fp32 [T, H*dv]; state: [slots][H][dv][DKP] fp32.  vec: four elements a load when staging.
template <typename TA>
__global__ void __launch_bounds__(THREADS, DK <= 128 ? 2 : 1)
gated_scan_kernel(const TA* __restrict__ q, int q_stride, const TA* __restrict__ k, int k_stride,
                  const TA* __restrict__ v, int v_stride, const float* __restrict__ alpha, int a_stride,
                  float q_scale, float* __restrict__ out,
                  float* __restrict__ state, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                  int H, int dv, int vec) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float smem[];
    constexpr int HALF = half_floats(3);
    const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
    const int tid = threadIdx.x;
    const bool loader = tid >= WORKERS;
    const int lt = tid - WORKERS;
    const int cg = tid / R, rg = tid % R;                    // of the computing threads: column group, lane in it
    const int t_begin = cu_q[b], t_end = cu_q[b + 1];
    const int rounds = (t_end - t_begin + TC - 1) / TC;
    if (DKP != DK) {                                         // rows beyond DK stay zero
        for (int e = tid; e < 2 * HALF; e += THREADS) smem[e] = 0.f;
        __syncthreads();
    }

    auto stage = [&](int round) {
        const GatedHalf hb(smem + (round & 1) * HALF);
        const int t0 = t_begin + round * TC, nt = min(TC, t_end - t0);
        float vv[PERV];
        load_values(vv, v, v_stride, t0, nt, h, dv, c0, lt);
        // every load of the round is issued before the first is used: addresses past the round's
        // end are clamped to its last element (read again, stored nowhere) so that no load is conditional
        if (vec) {
            float4 qv[PER4], kv[PER4], av[PER4];
#pragma unroll
            for (int j = 0; j < PER4; ++j) {
                const int e = min(lt + j * WORKERS, nt * (DK / 4) - 1);
                const int tok = e / (DK / 4), i = (e - tok * (DK / 4)) * 4;
                const size_t t = (size_t)(t0 + tok), c = (size_t)h * DK + i;
                qv[j] = ld4(q + t * q_stride + c);
                kv[j] = ld4(k + t * k_stride + c);
                av[j] = ld4(alpha + t * a_stride + c);
            }
#pragma unroll
            for (int j = 0; j < PER4; ++j) {
                const int e = lt + j * WORKERS;
                if (e < nt * (DK / 4)) {
                    const int tok = e / (DK / 4), i = (e - tok * (DK / 4)) * 4;
                    const int at = tok * ROWLEN + row_at(i);
                    *reinterpret_cast<float4*>(hb.q + at) = scaled(qv[j], q_scale);
                    *reinterpret_cast<float4*>(hb.k + at) = kv[j];
                    *reinterpret_cast<float4*>(hb.a + at) = av[j];
                }
            }
        } else {
            float qv[PER], kv[PER], av[PER];
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int e = min(lt + j * WORKERS, nt * DK - 1);
                const int tok = e / DK, i = e - tok * DK;
                const size_t t = (size_t)(t0 + tok), c = (size_t)h * DK + i;
                qv[j] = ld(q, t * q_stride + c);
                kv[j] = ld(k, t * k_stride + c);
                av[j] = alpha[t * a_stride + c];
            }
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int e = lt + j * WORKERS;
                if (e < nt * DK) {
                    const int tok = e / DK, i = e - tok * DK;
                    const int at = tok * ROWLEN + row_at(i);
                    hb.q[at] = qv[j] * q_scale;
                    hb.k[at] = kv[j];
                    hb.a[at] = av[j];
                }
            }
        }
        store_values(hb.v, vv, nt, dv, c0, lt);
    };

    bool ok[C];
#pragma unroll
    for (int j = 0; j < C; ++j) ok[j] = !loader && c0 + cg * C + j < dv;
    float* sp = nullptr;
    float S[C][NR];
    if (loader) {
        if (rounds > 0) stage(0);
    } else {
        sp = state + ((((size_t)state_slots[b] * H + h) * dv + c0 + cg * C) * DKP + rg * NR);
        load_state(S, sp, ok);
    }
    __syncthreads();
    for (int round = 0; round < rounds; ++round) {
        if (loader) {
            if (round + 1 < rounds) stage(round + 1);
        } else {
            const GatedHalf hb(smem + (round & 1) * HALF);
            const int t0 = t_begin + round * TC, nt = min(TC, t_end - t0);
            float* op = out + ((size_t)t0 * H + h) * dv + c0 + cg * C;
            if (nt == TC) {
                // the lanes' parts of TB tokens first, their sums after: a shuffle orders the
                // instructions around it, and a batch of them overlaps where one a token would not
#pragma unroll
                for (int tb = 0; tb < TC; tb += TB) {
                    GroupSums<TB * C> sums;                  // value i * C + j: token tb + i, column j
#pragma unroll
                    for (int i = 0; i < TB; ++i) {
                        float part[C];
                        gated_token(S, hb, tb + i, rg, cg, part);
#pragma unroll
                        for (int j = 0; j < C; ++j) sums.x[i * C + j] = part[j];
                    }
                    sums.run(rg);
                    if (sums.owner) {
#pragma unroll
                        for (int n = 0; n < TB * C; ++n) {
                            if (n < sums.count) {
                                const int idx = sums.first + n, i = idx / C, j = idx - i * C;
                                if (c0 + cg * C + j < dv) op[(size_t)(tb + i) * H * dv + j] = sums.x[n];
                            }
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int tok = 0; tok < nt; ++tok) {
                    float part[C];
                    gated_token(S, hb, tok, rg, cg, part);
#pragma unroll
                    for (int j = 0; j < C; ++j) {
                        const float o = group_sum(part[j]);
                        if (rg == 0 && ok[j]) op[(size_t)tok * H * dv + j] = o;
                    }
                }
            }
        }
        __syncthreads();
    }
    if (!loader) store_state(S, sp, ok);
}

// ------------------------------------------------------------------------------- delta
struct DeltaHalf {
    float *r, *k, *w, *u, *au, *v;
    __device__ DeltaHalf(float* base)
        : r(base), k(base + TC * ROWLEN), w(base + 2 * TC * ROWLEN), u(base + 3 * TC * ROWLEN),
          au(base + 4 * TC * ROWLEN), v(base + 5 * TC * ROWLEN) {}
};

__device__ __forceinline__ void delta_token(float (&S)[C][NR], const DeltaHalf& b, int tok, int rg, int cg, float (&part)[C]) {
    const int at = tok * ROWLEN + rg * NRP;
    const float4* u4 = reinterpret_cast<const float4*>(b.u + at);
    float d0[C], d1[C], dot[C];
#pragma unroll
    for (int j = 0; j < C; ++j) d0[j] = d1[j] = 0.f;
#pragma unroll
    for (int m = 0; m < NR / 4; ++m) {
        const float4 u = u4[m];
#pragma unroll
        for (int j = 0; j < C; ++j) dot_rows(&S[j][4 * m], u, d0[j], d1[j]);
    }
#pragma unroll
    for (int j = 0; j < C; ++j) dot[j] = d0[j] + d1[j];
    all_sums(dot, rg);
    const float4* w4 = reinterpret_cast<const float4*>(b.w + at);
    const float4* au4 = reinterpret_cast<const float4*>(b.au + at);
    const float4* k4 = reinterpret_cast<const float4*>(b.k + at);
    const float4* r4 = reinterpret_cast<const float4*>(b.r + at);
    float vj[C], o0[C], o1[C];
#pragma unroll
    for (int j = 0; j < C; ++j) {
        vj[j] = b.v[tok * COLS + cg * C + j];
        o0[j] = o1[j] = 0.f;
    }
#pragma unroll
    for (int m = 0; m < NR / 4; ++m) {
        const float4 w = w4[m], au = au4[m], kk = k4[m], rr = r4[m];
#pragma unroll
        for (int j = 0; j < C; ++j) delta_rows(&S[j][4 * m], w, au, kk, rr, dot[j], vj[j], o0[j], o1[j]);
    }
#pragma unroll
    for (int j = 0; j < C; ++j) part[j] = o0[j] + o1[j];
}

// r, k: [T, >= H*DK]; v: [T, >= H*dv]; w (decays), u (unit keys), au (removal rate times unit key):
// fp32 [T, H*DK] with one row stride.
template <typename TA>
__global__ void __launch_bounds__(THREADS, DK <= 128 ? 2 : 1)
delta_scan_kernel(const TA* __restrict__ r, int r_stride, const TA* __restrict__ k, int k_stride,
                  const TA* __restrict__ v, int v_stride, const float* __restrict__ w, const float* __restrict__ u,
                  const float* __restrict__ au, int f_stride, float* __restrict__ out,
                  float* __restrict__ state, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                  int H, int dv, int vec) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float smem[];
    constexpr int HALF = half_floats(5);
    const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
    const int tid = threadIdx.x;
    const bool loader = tid >= WORKERS;
    const int lt = tid - WORKERS;
    const int cg = tid / R, rg = tid % R;
    const int t_begin = cu_q[b], t_end = cu_q[b + 1];
    const int rounds = (t_end - t_begin + TC - 1) / TC;
    if (DKP != DK) {
        for (int e = tid; e < 2 * HALF; e += THREADS) smem[e] = 0.f;
        __syncthreads();
    }

    auto stage = [&](int round) {
        const DeltaHalf hb(smem + (round & 1) * HALF);
        const int t0 = t_begin + round * TC, nt = min(TC, t_end - t0);
        float vv[PERV];
        load_values(vv, v, v_stride, t0, nt, h, dv, c0, lt);
        if (vec) {                                           // loads unconditional, as in the gated kernel
            float4 rv[PER4], kv[PER4], wv[PER4], uv[PER4], av[PER4];
#pragma unroll
            for (int j = 0; j < PER4; ++j) {
                const int e = min(lt + j * WORKERS, nt * (DK / 4) - 1);
                const int tok = e / (DK / 4), i = (e - tok * (DK / 4)) * 4;
                const size_t t = (size_t)(t0 + tok), c = (size_t)h * DK + i;
                rv[j] = ld4(r + t * r_stride + c);
                kv[j] = ld4(k + t * k_stride + c);
                wv[j] = ld4(w + t * f_stride + c);
                uv[j] = ld4(u + t * f_stride + c);
                av[j] = ld4(au + t * f_stride + c);
            }
#pragma unroll
            for (int j = 0; j < PER4; ++j) {
                const int e = lt + j * WORKERS;
                if (e < nt * (DK / 4)) {
                    const int tok = e / (DK / 4), i = (e - tok * (DK / 4)) * 4;
                    const int at = tok * ROWLEN + row_at(i);
                    *reinterpret_cast<float4*>(hb.r + at) = rv[j];
                    *reinterpret_cast<float4*>(hb.k + at) = kv[j];
                    *reinterpret_cast<float4*>(hb.w + at) = wv[j];
                    *reinterpret_cast<float4*>(hb.u + at) = uv[j];
                    *reinterpret_cast<float4*>(hb.au + at) = av[j];
                }
            }
        } else {
            float rv[PER], kv[PER], wv[PER], uv[PER], av[PER];
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int e = min(lt + j * WORKERS, nt * DK - 1);
                const int tok = e / DK, i = e - tok * DK;
                const size_t t = (size_t)(t0 + tok), c = (size_t)h * DK + i;
                rv[j] = ld(r, t * r_stride + c);
                kv[j] = ld(k, t * k_stride + c);
                wv[j] = w[t * f_stride + c];
                uv[j] = u[t * f_stride + c];
                av[j] = au[t * f_stride + c];
            }
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const int e = lt + j * WORKERS;
                if (e < nt * DK) {
                    const int tok = e / DK, i = e - tok * DK;
                    const int at = tok * ROWLEN + row_at(i);
                    hb.r[at] = rv[j];
                    hb.k[at] = kv[j];
                    hb.w[at] = wv[j];
                    hb.u[at] = uv[j];
                    hb.au[at] = av[j];
                }
            }
        }
        store_values(hb.v, vv, nt, dv, c0, lt);
    };

    bool ok[C];
#pragma unroll
    for (int j = 0; j < C; ++j) ok[j] = !loader && c0 + cg * C + j < dv;
    float* sp = nullptr;
    float S[C][NR];
    if (loader) {
        if (rounds > 0) stage(0);
    } else {
        sp = state + ((((size_t)state_slots[b] * H + h) * dv + c0 + cg * C) * DKP + rg * NR);
        load_state(S, sp, ok);
    }
    __syncthreads();
    for (int round = 0; round < rounds; ++round) {
        if (loader) {
            if (round + 1 < rounds) stage(round + 1);
        } else {
            const DeltaHalf hb(smem + (round & 1) * HALF);
            const int t0 = t_begin + round * TC, nt = min(TC, t_end - t0);
            float* op = out + ((size_t)t0 * H + h) * dv + c0 + cg * C;
            if (nt == TC) {
#pragma unroll
                for (int tb = 0; tb < TC; tb += TB) {        // the outputs' sums in batches, as in the gated kernel
                    GroupSums<TB * C> sums;                  // value i * C + j: token tb + i, column j
#pragma unroll
                    for (int i = 0; i < TB; ++i) {
                        float part[C];
                        delta_token(S, hb, tb + i, rg, cg, part);
#pragma unroll
                        for (int j = 0; j < C; ++j) sums.x[i * C + j] = part[j];
                    }
                    sums.run(rg);
                    if (sums.owner) {
#pragma unroll
                        for (int n = 0; n < TB * C; ++n) {
                            if (n < sums.count) {
                                const int idx = sums.first + n, i = idx / C, j = idx - i * C;
                                if (c0 + cg * C + j < dv) op[(size_t)(tb + i) * H * dv + j] = sums.x[n];
                            }
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int tok = 0; tok < nt; ++tok) {
                    float part[C];
                    delta_token(S, hb, tok, rg, cg, part);
#pragma unroll
                    for (int j = 0; j < C; ++j) {
                        const float o = group_sum(part[j]);
                        if (rg == 0 && ok[j]) op[(size_t)tok * H * dv + j] = o;
                    }
                }
            }
        }
        __syncthreads();
    }
    if (!loader) store_state(S, sp, ok);
}

// ------------------------------------------------------------- entries of a single token
// A step in which every entry brings one token (decoding): no rounds and no staging.  A CTA of
// WORKERS threads owns COLS value channels of one head of one entry; a lane reads its rows of the
// token's vectors straight from global memory and does the same arithmetic in the same order as
// the walk above, so a token's bits do not depend on which kernel took it.
template <typename TA>
__device__ __forceinline__ void rows_of(float4 (&x)[NR / 4], const TA* p, int rg, float scale) {
#pragma unroll
    for (int m = 0; m < NR / 4; ++m) {
        float e[4];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            const int i = rg * NR + 4 * m + n;
            e[n] = i < DK ? to_f32<TA>(p[i]) * scale : 0.f;
        }
        x[m] = make_float4(e[0], e[1], e[2], e[3]);
    }
}

template <typename TA>
__global__ void __launch_bounds__(WORKERS)
gated_step_kernel(const TA* __restrict__ q, int q_stride, const TA* __restrict__ k, int k_stride,
                  const TA* __restrict__ v, int v_stride, const float* __restrict__ alpha, int a_stride,
                  float q_scale, float* __restrict__ out, float* __restrict__ state,
                  const int* __restrict__ cu_q, const int* __restrict__ state_slots, int H, int dv) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
    const int cg = threadIdx.x / R, rg = threadIdx.x % R;
    const int t = cu_q[b];
    if (cu_q[b + 1] - t != 1) return;                        // the host sends only steps of single tokens here
    bool ok[C];
#pragma unroll
    for (int j = 0; j < C; ++j) ok[j] = c0 + cg * C + j < dv;
    float* sp = state + ((((size_t)state_slots[b] * H + h) * dv + c0 + cg * C) * DKP + rg * NR);
    float S[C][NR];
    load_state(S, sp, ok);
    float4 a[NR / 4], kk[NR / 4], qq[NR / 4];
    rows_of(a, alpha + (size_t)t * a_stride + (size_t)h * DK, rg, 1.f);
    rows_of(kk, k + (size_t)t * k_stride + (size_t)h * DK, rg, 1.f);
    rows_of(qq, q + (size_t)t * q_stride + (size_t)h * DK, rg, q_scale);
#pragma unroll
    for (int j = 0; j < C; ++j) {
        const float vj = ok[j] ? to_f32<TA>(v[(size_t)t * v_stride + (size_t)h * dv + c0 + cg * C + j]) : 0.f;
        float o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int m = 0; m < NR / 4; ++m) gated_rows(&S[j][4 * m], a[m], kk[m], qq[m], vj, o0, o1);
        const float o = group_sum(o0 + o1);
        if (rg == 0 && ok[j]) out[((size_t)t * H + h) * dv + c0 + cg * C + j] = o;
    }
    store_state(S, sp, ok);
}

template <typename TA>
__global__ void __launch_bounds__(WORKERS)
delta_step_kernel(const TA* __restrict__ r, int r_stride, const TA* __restrict__ k, int k_stride,
                  const TA* __restrict__ v, int v_stride, const float* __restrict__ w, const float* __restrict__ u,
                  const float* __restrict__ au, int f_stride, float* __restrict__ out, float* __restrict__ state,
                  const int* __restrict__ cu_q, const int* __restrict__ state_slots, int H, int dv) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
    const int cg = threadIdx.x / R, rg = threadIdx.x % R;
    const int t = cu_q[b];
    if (cu_q[b + 1] - t != 1) return;
    bool ok[C];
#pragma unroll
    for (int j = 0; j < C; ++j) ok[j] = c0 + cg * C + j < dv;
    float* sp = state + ((((size_t)state_slots[b] * H + h) * dv + c0 + cg * C) * DKP + rg * NR);
    float S[C][NR];
    load_state(S, sp, ok);
    const size_t f = (size_t)t * f_stride + (size_t)h * DK;
    float4 uu[NR / 4], ww[NR / 4], aa[NR / 4], kk[NR / 4], rr[NR / 4];
    rows_of(uu, u + f, rg, 1.f);
    rows_of(ww, w + f, rg, 1.f);
    rows_of(aa, au + f, rg, 1.f);
    rows_of(kk, k + (size_t)t * k_stride + (size_t)h * DK, rg, 1.f);
    rows_of(rr, r + (size_t)t * r_stride + (size_t)h * DK, rg, 1.f);
#pragma unroll
    for (int j = 0; j < C; ++j) {
        float d0 = 0.f, d1 = 0.f;
#pragma unroll
        for (int m = 0; m < NR / 4; ++m) dot_rows(&S[j][4 * m], uu[m], d0, d1);
        const float dot = group_sum(d0 + d1);
        const float vj = ok[j] ? to_f32<TA>(v[(size_t)t * v_stride + (size_t)h * dv + c0 + cg * C + j]) : 0.f;
        float o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int m = 0; m < NR / 4; ++m) delta_rows(&S[j][4 * m], ww[m], aa[m], kk[m], rr[m], dot, vj, o0, o1);
        const float o = group_sum(o0 + o1);
        if (rg == 0 && ok[j]) out[((size_t)t * H + h) * dv + c0 + cg * C + j] = o;
    }
    store_state(S, sp, ok);
}

inline bool aligned4(const void* p, int esize) { return (reinterpret_cast<uintptr_t>(p) % (4 * (size_t)esize)) == 0; }

template <typename Kernel>
int allow_shared(Kernel kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return 0;
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}
}  // namespace

RI_API int ri_recurrent_key_dim() { return DK; }
RI_API int ri_recurrent_state_rows() { return DKP; }

// `single` != 0: every entry brings exactly one token (the kernel without staging takes the step)
RI_API int ri_gated_scan(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride,
                         const float* alpha, int a_stride, int act_dtype, float q_scale, float* out, float* state,
                         const int* cu_q, const int* state_slots, int entries, int H, int dv, int single,
                         void* stream) {
    if (entries <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((dv + COLS - 1) / COLS, H, entries);
    const size_t smem = 2 * (size_t)half_floats(3) * sizeof(float);
    const int esize = act_dtype == RI_BF16 ? 2 : 4;
    const int vec = DK % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && a_stride % 4 == 0 &&
                    aligned4(q, esize) && aligned4(k, esize) && aligned4(alpha, 4);
#define RI_GS(TA) do { \
    if (single) { \
        RI_CHECKED(ri_launch(gated_step_kernel<TA>, grid, dim3(WORKERS), 0, s, (const TA*)q, q_stride, (const TA*)k, \
            k_stride, (const TA*)v, v_stride, alpha, a_stride, q_scale, out, state, cu_q, state_slots, H, dv)); \
        break; \
    } \
    static bool allowed = false; \
    if (!allowed) { RI_CHECKED(allow_shared(gated_scan_kernel<TA>, smem)); allowed = true; } \
    RI_CHECKED(ri_launch(gated_scan_kernel<TA>, grid, dim3(THREADS), smem, s, (const TA*)q, q_stride, \
        (const TA*)k, k_stride, (const TA*)v, v_stride, alpha, a_stride, q_scale, out, state, \
        cu_q, state_slots, H, dv, vec)); } while (0)
    if (act_dtype == RI_BF16) RI_GS(bf16);
    else RI_GS(float);
#undef RI_GS
    return ri_launch_status();
}

RI_API int ri_delta_scan(const void* r, int r_stride, const void* k, int k_stride, const void* v, int v_stride,
                         const float* w, const float* u, const float* au, int f_stride, int act_dtype,
                         float* out, float* state, const int* cu_q, const int* state_slots, int entries, int H,
                         int dv, int single, void* stream) {
    if (entries <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((dv + COLS - 1) / COLS, H, entries);
    const size_t smem = 2 * (size_t)half_floats(5) * sizeof(float);
    const int esize = act_dtype == RI_BF16 ? 2 : 4;
    const int vec = DK % 4 == 0 && r_stride % 4 == 0 && k_stride % 4 == 0 && f_stride % 4 == 0 &&
                    aligned4(r, esize) && aligned4(k, esize) && aligned4(w, 4) && aligned4(u, 4) && aligned4(au, 4);
#define RI_DS(TA) do { \
    if (single) { \
        RI_CHECKED(ri_launch(delta_step_kernel<TA>, grid, dim3(WORKERS), 0, s, (const TA*)r, r_stride, (const TA*)k, \
            k_stride, (const TA*)v, v_stride, w, u, au, f_stride, out, state, cu_q, state_slots, H, dv)); \
        break; \
    } \
    static bool allowed = false; \
    if (!allowed) { RI_CHECKED(allow_shared(delta_scan_kernel<TA>, smem)); allowed = true; } \
    RI_CHECKED(ri_launch(delta_scan_kernel<TA>, grid, dim3(THREADS), smem, s, (const TA*)r, r_stride, \
        (const TA*)k, k_stride, (const TA*)v, v_stride, w, u, au, f_stride, out, state, cu_q, state_slots, H, dv, vec)); \
    } while (0)
    if (act_dtype == RI_BF16) RI_DS(bf16);
    else RI_DS(float);
#undef RI_DS
    return ri_launch_status();
}

RI_API void ri_set_pdl(int on) { ri_pdl_flag() = on ? 1 : 0; }
