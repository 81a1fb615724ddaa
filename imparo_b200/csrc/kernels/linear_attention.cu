// Linear attention with a per-head decay, as a recurrence over a fixed-size state:
//
//     S_t = decay_h * S_(t-1) + k_t v_t^T        (S: [dim, vdim] per head, 32-bit, one per request slot)
//     o_t = S_t^T q_t
//
// with q, k, v = act(projection) (act = SiLU or none), for ragged batches: a request's rows are walked in
// order from the state its slot holds, and the state is written back at the end, so a prompt cut into
// portions, or decoded token by token, runs the same sequence of operations as the whole prompt.
//
// recurrent kernel: one warp per (request, head, 32 value columns).  A lane owns one column of the state in
// registers (dim values); the request's rows are staged 16 at a time in shared memory (activated, 32-bit),
// then each row costs dim multiply-adds for the state and dim for the output.  Everything that enters the
// recurrence is 32-bit; only the projections are read in the activations' dtype.
#include "common.cuh"
#include <mma.h>

namespace imparo {

constexpr int LA_STAGE = 16;

// Rows [r_begin, r_end) of one request and head through the recurrence, for the 32 value columns of this warp.
// S: this lane's column of the state (dim values, in registers).  out: null when only the state is wanted.
template <typename T, int DMAX, bool SILU>
__device__ __forceinline__ void la_walk(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, size_t row_stride,
                                        float dec, float (&S)[DMAX], int r_begin, int r_end, float* __restrict__ out,
                                        int h, int heads, int dim, int vdim, int col, bool live,
                                        float (*qs)[DMAX], float (*ks)[DMAX], float (*vs)[32]) {
    const int lane = threadIdx.x;
    for (int base = r_begin; base < r_end; base += LA_STAGE) {
        const int n = min(LA_STAGE, r_end - base);
        __syncwarp();
        for (int r = 0; r < n; ++r) {
            const T* qr = q + (size_t)(base + r) * row_stride + (size_t)h * dim;
            const T* kr = k + (size_t)(base + r) * row_stride + (size_t)h * dim;
            for (int d = lane; d < DMAX; d += 32) {
                float a = 0.f, b = 0.f;
                if (d < dim) {
                    b = to_f32(kr[d]);
                    if (SILU) b = silu(b);
                    if (out) { a = to_f32(qr[d]); if (SILU) a = silu(a); }
                }
                qs[r][d] = a; ks[r][d] = b;
            }
            float c = 0.f;
            if (live) {
                c = to_f32(v[(size_t)(base + r) * row_stride + (size_t)h * vdim + col]);
                if (SILU) c = silu(c);
            }
            vs[r][lane] = c;
        }
        __syncwarp();
        for (int r = 0; r < n; ++r) {
            const float vv = vs[r][lane];
            float o = 0.f;
#pragma unroll
            for (int d = 0; d < DMAX; d += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(&ks[r][d]);
                const float4 q4 = *reinterpret_cast<const float4*>(&qs[r][d]);
                S[d] = dec * S[d] + k4.x * vv;         o += S[d] * q4.x;
                S[d + 1] = dec * S[d + 1] + k4.y * vv; o += S[d + 1] * q4.y;
                S[d + 2] = dec * S[d + 2] + k4.z * vv; o += S[d + 2] * q4.z;
                S[d + 3] = dec * S[d + 3] + k4.w * vv; o += S[d + 3] * q4.w;
            }
            if (out && live) out[(size_t)(base + r) * ((size_t)heads * vdim) + (size_t)h * vdim + col] = o;
        }
    }
}

template <typename T, int DMAX, bool SILU>
__global__ void __launch_bounds__(32)
linear_attention_recurrent_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, size_t row_stride,
                                  const float* __restrict__ decay, float* __restrict__ state,
                                  const int* __restrict__ item_row_start, const int* __restrict__ item_slot, int n_slots,
                                  float* __restrict__ out, int heads, int dim, int vdim, int* status) {
    __shared__ __align__(16) float qs[LA_STAGE][DMAX], ks[LA_STAGE][DMAX], vs[LA_STAGE][32];
    pdl_trigger();
    const int item = blockIdx.x, h = blockIdx.y, col = blockIdx.z * 32 + threadIdx.x;
    const int lane = threadIdx.x;
    const int r0 = item_row_start[item], r1 = item_row_start[item + 1];
    const int slot = item_slot[item];
    const float dec = decay[h];
    pdl_wait();
    if (slot < 0 || slot >= n_slots) {
        if (lane == 0) report(status, IMPARO_ST_SLOT_RANGE, 43, item, slot);
        return;
    }
    const bool live = col < vdim;
    float* sp = state + (((size_t)slot * heads + h) * dim) * vdim + col;
    float S[DMAX];
#pragma unroll
    for (int d = 0; d < DMAX; ++d) S[d] = (live && d < dim) ? sp[(size_t)d * vdim] : 0.f;
    la_walk<T, DMAX, SILU>(q, k, v, row_stride, dec, S, r0, r1, out, h, heads, dim, vdim, col, live, qs, ks, vs);
    if (live) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d) if (d < dim) sp[(size_t)d * vdim] = S[d];
    }
}

// ---- long portions: the same recurrence, cut into chunks of `chunk` rows that run side by side ---------------
// A request's rows are cut into chunks (chunk c of a request: rows r0 + c*chunk ...); the chunks of all requests of
// the launch are numbered in order.  Three launches:
//   local: every chunk alone, from a zero state: L_c = sum_j decay^(n-1-j) k_j v_j^T  -> chunk_state[c]
//   scan:  per request, over its chunks in order: chunk_state[c] becomes the state the chunk starts from
//          (s, beginning with the slot's state), s = decay^n_c * s + L_c; at the end the slot's state = s
//   out:   every chunk alone from its starting state: the outputs of its rows
// All of it in 32-bit on the CUDA cores: the result differs from the row-by-row walk by the order of additions only.
// The grid's x extent is an upper bound of the number of chunks (rows / chunk + requests); blocks beyond it return.
__device__ __forceinline__ bool la_find_chunk(const int* __restrict__ item_row_start, int n_items, int chunk, int g,
                                              int& item, int& r_begin, int& r_end) {
    int basec = 0;
    for (int i = 0; i < n_items; ++i) {
        const int r0 = item_row_start[i], r1 = item_row_start[i + 1];
        const int nc = (r1 - r0 + chunk - 1) / chunk;
        if (g < basec + nc) {
            item = i;
            r_begin = r0 + (g - basec) * chunk;
            r_end = min(r_begin + chunk, r1);
            return true;
        }
        basec += nc;
    }
    return false;
}

template <typename T, int DMAX, bool SILU, bool OUT>
__global__ void __launch_bounds__(32)
linear_attention_chunk_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, size_t row_stride,
                              const float* __restrict__ decay, float* __restrict__ chunk_state,
                              const int* __restrict__ item_row_start, int n_items, int chunk,
                              float* __restrict__ out, int heads, int dim, int vdim) {
    __shared__ __align__(16) float qs[LA_STAGE][DMAX], ks[LA_STAGE][DMAX], vs[LA_STAGE][32];
    pdl_trigger();
    const int g = blockIdx.x, h = blockIdx.y, col = blockIdx.z * 32 + threadIdx.x;
    int item, r_begin, r_end;
    const bool found = la_find_chunk(item_row_start, n_items, chunk, g, item, r_begin, r_end);
    const float dec = decay[h];
    pdl_wait();
    if (!found) return;
    const bool live = col < vdim;
    float* sp = chunk_state + (((size_t)g * heads + h) * dim) * vdim + col;
    float S[DMAX];
#pragma unroll
    for (int d = 0; d < DMAX; ++d) S[d] = (OUT && live && d < dim) ? sp[(size_t)d * vdim] : 0.f;
    la_walk<T, DMAX, SILU>(q, k, v, row_stride, dec, S, r_begin, r_end, OUT ? out : nullptr, h, heads, dim, vdim, col, live, qs, ks, vs);
    if (!OUT && live) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d) if (d < dim) sp[(size_t)d * vdim] = S[d];
    }
}

// grid (requests, heads, ceil(dim*vdim / 256)); one state element per thread, the request's chunks in order
__global__ void __launch_bounds__(256)
linear_attention_scan_kernel(const float* __restrict__ decay, float* __restrict__ chunk_state, float* __restrict__ state,
                             const int* __restrict__ item_row_start, const int* __restrict__ item_slot, int n_items, int n_slots,
                             int chunk, int heads, int per_head, int* status) {
    pdl_trigger();
    const int item = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * 256 + threadIdx.x;
    int first = 0;
    for (int i = 0; i < item; ++i) first += (item_row_start[i + 1] - item_row_start[i] + chunk - 1) / chunk;
    const int r0 = item_row_start[item], r1 = item_row_start[item + 1];
    const int slot = item_slot[item];
    const float dec = decay[h];
    pdl_wait();
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0 && blockIdx.z == 0) report(status, IMPARO_ST_SLOT_RANGE, 44, item, slot);
        return;
    }
    if (e >= per_head) return;
    float* sp = state + ((size_t)slot * heads + h) * per_head + e;
    float s = *sp;
    const float dec_full = powf(dec, (float)chunk);
    const int nc = (r1 - r0 + chunk - 1) / chunk;
    const size_t cstride = (size_t)heads * per_head;
    float* cp = chunk_state + ((size_t)first * heads + h) * per_head + e;
    for (int c0 = 0; c0 < nc; c0 += 8) {                      // eight chunks' sums requested together, then the chain
        float loc[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) loc[u] = c0 + u < nc ? __ldcg(cp + (size_t)(c0 + u) * cstride) : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (c0 + u < nc) {
                const int n = min(chunk, r1 - r0 - (c0 + u) * chunk);
                cp[(size_t)(c0 + u) * cstride] = s;
                s = (n == chunk ? dec_full : powf(dec, (float)n)) * s + loc[u];
            }
        }
    }
    *sp = s;
}


// ---- the chunks on tensor cores (bfloat16, key and value sizes multiples of 16 up to 128, chunks of 64 rows) ----
// With Q, K [64, dim] and V [64, vdim] the chunk's activated rows (bfloat16) and d the head's decay:
//   local:  L = sum_j d^(n-1-j) k_j v_j^T = Kd^T V, Kd_j = d^(n-1-j) k_j formed in 32-bit and fed to the tensor cores as the
//           sum of two bfloat16 numbers (a high and a low part: two products), so that the decays are not rounded to 8 bits
//   out:    o_i = sum_(j<=i) (q_i.k_j) d^(i-j) v_j + d^(i+1) (S0^T q_i):  scores Q K^T accumulated in 32-bit, multiplied by the
//           decay powers in 32-bit, rounded to bfloat16 for the product with V (as a softmax's weights are); the state the
//           chunk starts from enters as a high and a low bfloat16 part (two products) and its rows' decay d^(i+1) multiplies
//           the 32-bit result.  The state itself is only ever added to in 32-bit (the scan).
// One CTA of four warps per (chunk, head); wmma fragments of 16 x 16 x 16 (mma.sync); operands staged in padded shared memory.
namespace lt {
namespace wm = nvcuda::wmma;
constexpr int C = 64, PAD = 8, THREADS = 256;
using bf16 = __nv_bfloat16;

__device__ __forceinline__ bool find_chunk(const int* __restrict__ item_row_start, int n_items, int g, int& r_begin, int& r_end) {
    int item;
    return la_find_chunk(item_row_start, n_items, C, g, item, r_begin, r_end);
}

// rows [r_begin, r_begin + n) x `width` columns at `src` (row stride in elements) -> dst [C][ld] (and lo [C][ld]): activated,
// times factor(row) in 32-bit, as a bfloat16 high part (and the low part of what that rounding lost); rows from n on are zero
template <bool SILU, bool SPLIT, typename F>
__device__ __forceinline__ void stage(const bf16* __restrict__ src, size_t row_stride, int r_begin, int n, int width,
                                      bf16* __restrict__ dst, bf16* __restrict__ lo, int ld, F factor) {
    const int vecs = width / 8;
    constexpr int U = 4;                                      // loads requested together per thread
    for (int base = threadIdx.x; base < C * vecs; base += THREADS * U) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = base + u * THREADS;
            const int r = idx / vecs, c = (idx - r * vecs) * 8;
            raw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (idx < C * vecs && r < n) raw[u] = *reinterpret_cast<const uint4*>(src + (size_t)(r_begin + r) * row_stride + c);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = base + u * THREADS;
            if (idx >= C * vecs) break;
            const int r = idx / vecs, c = (idx - r * vecs) * 8;
            uint4 hi4 = make_uint4(0u, 0u, 0u, 0u), lo4 = hi4;
            if (r < n) {
                const bf16* e = reinterpret_cast<const bf16*>(&raw[u]);
                const float f = factor(r);
                bf16* ho = reinterpret_cast<bf16*>(&hi4);
                bf16* lw = reinterpret_cast<bf16*>(&lo4);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float x = __bfloat162float(e[q]);
                    if (SILU) x = silu_bf16(x);
                    x *= f;
                    ho[q] = __float2bfloat16_rn(x);
                    if (SPLIT) lw[q] = __float2bfloat16_rn(x - __bfloat162float(ho[q]));
                }
            }
            *reinterpret_cast<uint4*>(dst + (size_t)r * ld + c) = hi4;
            if (SPLIT) *reinterpret_cast<uint4*>(lo + (size_t)r * ld + c) = lo4;
        }
    }
}

template <bool SILU>
__global__ void __launch_bounds__(THREADS)
local_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v, size_t row_stride, const float* __restrict__ decay,
             float* __restrict__ chunk_state, const int* __restrict__ item_row_start, int n_items, int heads, int dim, int vdim) {
    extern __shared__ __align__(128) unsigned char lt_smem[];
    __shared__ float pw[C + 1];
    pdl_trigger();
    const int g = blockIdx.x, h = blockIdx.y;
    int r_begin, r_end;
    const bool found = find_chunk(item_row_start, n_items, g, r_begin, r_end);
    const float dec = decay[h];
    if (threadIdx.x <= C) pw[threadIdx.x] = powf(dec, (float)threadIdx.x);
    pdl_wait();
    if (!found) return;
    const int n = r_end - r_begin;
    const int ldk = dim + PAD, ldv = vdim + PAD;
    bf16* k_hi = reinterpret_cast<bf16*>(lt_smem);
    bf16* k_lo = k_hi + C * ldk;
    bf16* v_s = k_lo + C * ldk;
    __syncthreads();
    stage<SILU, true>(k + (size_t)h * dim, row_stride, r_begin, n, dim, k_hi, k_lo, ldk, [&](int r) { return pw[n - 1 - r]; });
    stage<SILU, false>(v + (size_t)h * vdim, row_stride, r_begin, n, vdim, v_s, nullptr, ldv, [](int) { return 1.f; });
    __syncthreads();
    const int warp = threadIdx.x >> 5;
    const int dts = dim / 16, vts = vdim / 16;
    float* dst = chunk_state + ((size_t)g * heads + h) * dim * vdim;
    const int steps = (n + 15) / 16;                          // rows from n on are zero
    for (int t = warp; t < dts * vts; t += THREADS / 32) {
        const int dt = t / vts, vt = t - dt * vts;
        wm::fragment<wm::accumulator, 16, 16, 16, float> acc;
        wm::fill_fragment(acc, 0.f);
        for (int jj = 0; jj < steps; ++jj) {
            wm::fragment<wm::matrix_a, 16, 16, 16, bf16, wm::col_major> a_hi, a_lo;      // (d, j) at [j * ld + d]
            wm::fragment<wm::matrix_b, 16, 16, 16, bf16, wm::row_major> b;
            wm::load_matrix_sync(a_hi, k_hi + (size_t)jj * 16 * ldk + dt * 16, ldk);
            wm::load_matrix_sync(a_lo, k_lo + (size_t)jj * 16 * ldk + dt * 16, ldk);
            wm::load_matrix_sync(b, v_s + (size_t)jj * 16 * ldv + vt * 16, ldv);
            wm::mma_sync(acc, a_hi, b, acc);
            wm::mma_sync(acc, a_lo, b, acc);
        }
        wm::store_matrix_sync(dst + (size_t)dt * 16 * vdim + vt * 16, acc, vdim, wm::mem_row_major);
    }
}

template <bool SILU>
__global__ void __launch_bounds__(THREADS)
out_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, size_t row_stride,
           const float* __restrict__ decay, const float* __restrict__ chunk_state, const int* __restrict__ item_row_start,
           int n_items, float* __restrict__ out, int heads, int dim, int vdim) {
    extern __shared__ __align__(128) unsigned char lt_smem[];
    __shared__ float pw[C + 1];
    pdl_trigger();
    const int g = blockIdx.x, h = blockIdx.y;
    int r_begin, r_end;
    const bool found = find_chunk(item_row_start, n_items, g, r_begin, r_end);
    const float dec = decay[h];
    if (threadIdx.x <= C) pw[threadIdx.x] = powf(dec, (float)threadIdx.x);
    pdl_wait();
    if (!found) return;
    const int n = r_end - r_begin;
    // the value columns are shared out over the grid's z extent (each CTA computes the chunk's scores itself): half the
    // state and half of v per CTA, so that two CTAs fit an SM
    const int vcols = vdim / (int)gridDim.z, v0 = (int)blockIdx.z * vcols;
    const int ldq = dim + PAD, ldv = vcols + PAD, lds = vcols + PAD, ldab = C + PAD, ldp = 20;
    bf16* q_s = reinterpret_cast<bf16*>(lt_smem);
    bf16* k_s = q_s + C * ldq;
    bf16* v_s = k_s + C * ldq;
    bf16* s_hi = v_s + C * ldv;
    bf16* s_lo = s_hi + dim * lds;
    bf16* a_bf = s_lo + dim * lds;
    float* patch = reinterpret_cast<float*>(a_bf + C * ldab) + (threadIdx.x >> 5) * 16 * ldp;
    auto one = [](int) { return 1.f; };
    stage<SILU, false>(q + (size_t)h * dim, row_stride, r_begin, n, dim, q_s, nullptr, ldq, one);
    stage<SILU, false>(k + (size_t)h * dim, row_stride, r_begin, n, dim, k_s, nullptr, ldq, one);
    stage<SILU, false>(v + (size_t)h * vdim + v0, row_stride, r_begin, n, vcols, v_s, nullptr, ldv, one);
    {
        const float* src = chunk_state + ((size_t)g * heads + h) * dim * vdim + v0;
        const int vecs = vcols / 4;
        constexpr int U = 8;
        for (int base = threadIdx.x; base < dim * vecs; base += THREADS * U) {
            float4 xs[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * THREADS;
                const int r = idx / vecs, c = (idx - r * vecs) * 4;
                xs[u] = idx < dim * vecs ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)r * vdim + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * THREADS;
                if (idx >= dim * vecs) break;
                const int r = idx / vecs, c = (idx - r * vecs) * 4;
                const float4 x = xs[u];
                const __nv_bfloat162 h01 = __floats2bfloat162_rn(x.x, x.y), h23 = __floats2bfloat162_rn(x.z, x.w);
                const float2 f01 = __bfloat1622float2(h01), f23 = __bfloat1622float2(h23);
                const __nv_bfloat162 l01 = __floats2bfloat162_rn(x.x - f01.x, x.y - f01.y), l23 = __floats2bfloat162_rn(x.z - f23.x, x.w - f23.y);
                *reinterpret_cast<uint2*>(s_hi + (size_t)r * lds + c) = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
                *reinterpret_cast<uint2*>(s_lo + (size_t)r * lds + c) = make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
            }
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kts = dim / 16, vts = vcols / 16;
    // scores of the tiles on and below the diagonal: (0,0) (1,0) (1,1) (2,0) ... (3,3); each goes through the warp's patch,
    // where it is multiplied by the decay powers in 32-bit and masked, into the bfloat16 operand of the product with v
    for (int t = warp; t < 10; t += THREADS / 32) {
        int it = 0, jt = t;
        while (jt > it) { jt -= it + 1; ++it; }
        wm::fragment<wm::accumulator, 16, 16, 16, float> acc;
        wm::fill_fragment(acc, 0.f);
        for (int kk = 0; kk < kts; ++kk) {
            wm::fragment<wm::matrix_a, 16, 16, 16, bf16, wm::row_major> a;
            wm::fragment<wm::matrix_b, 16, 16, 16, bf16, wm::col_major> b;               // (d, j) at [j * ld + d]
            wm::load_matrix_sync(a, q_s + (size_t)it * 16 * ldq + kk * 16, ldq);
            wm::load_matrix_sync(b, k_s + (size_t)jt * 16 * ldq + kk * 16, ldq);
            wm::mma_sync(acc, a, b, acc);
        }
        wm::store_matrix_sync(patch, acc, ldp, wm::mem_row_major);
        __syncwarp();
        for (int e = lane; e < 256; e += 32) {
            const int i = it * 16 + (e >> 4), j = jt * 16 + (e & 15);
            const float w = (j <= i && i < n) ? patch[(e >> 4) * ldp + (e & 15)] * pw[i - j] : 0.f;
            a_bf[(size_t)i * ldab + j] = __float2bfloat16_rn(w);
        }
        __syncwarp();
    }
    __syncthreads();
    for (int t = warp; t < 4 * vts; t += THREADS / 32) {
        const int it = t & 3, vt = t >> 2;
        wm::fragment<wm::accumulator, 16, 16, 16, float> acc;
        wm::fill_fragment(acc, 0.f);
        for (int kk = 0; kk < kts; ++kk) {                   // the state the chunk starts from: S0^T q, high and low part
            wm::fragment<wm::matrix_a, 16, 16, 16, bf16, wm::row_major> a;
            wm::fragment<wm::matrix_b, 16, 16, 16, bf16, wm::row_major> b_hi, b_lo;
            wm::load_matrix_sync(a, q_s + (size_t)it * 16 * ldq + kk * 16, ldq);
            wm::load_matrix_sync(b_hi, s_hi + (size_t)kk * 16 * lds + vt * 16, lds);
            wm::load_matrix_sync(b_lo, s_lo + (size_t)kk * 16 * lds + vt * 16, lds);
            wm::mma_sync(acc, a, b_hi, acc);
            wm::mma_sync(acc, a, b_lo, acc);
        }
        wm::store_matrix_sync(patch, acc, ldp, wm::mem_row_major);
        __syncwarp();
        for (int e = lane; e < 256; e += 32) patch[(e >> 4) * ldp + (e & 15)] *= pw[it * 16 + (e >> 4) + 1];
        __syncwarp();
        wm::load_matrix_sync(acc, patch, ldp, wm::mem_row_major);
        for (int jj = 0; jj <= it; ++jj) {                    // the chunk's own rows up to the diagonal
            wm::fragment<wm::matrix_a, 16, 16, 16, bf16, wm::row_major> a;
            wm::fragment<wm::matrix_b, 16, 16, 16, bf16, wm::row_major> b;
            wm::load_matrix_sync(a, a_bf + (size_t)it * 16 * ldab + jj * 16, ldab);
            wm::load_matrix_sync(b, v_s + (size_t)jj * 16 * ldv + vt * 16, ldv);
            wm::mma_sync(acc, a, b, acc);
        }
        __syncwarp();
        wm::store_matrix_sync(patch, acc, ldp, wm::mem_row_major);
        __syncwarp();
        for (int e = lane; e < 256; e += 32) {
            const int r = it * 16 + (e >> 4);
            if (r < n) out[(size_t)(r_begin + r) * ((size_t)heads * vdim) + (size_t)h * vdim + v0 + vt * 16 + (e & 15)] = patch[(e >> 4) * ldp + (e & 15)];
        }
        __syncwarp();
    }
}

static size_t local_smem(int dim, int vdim) { return (size_t)C * (2 * (dim + PAD) + (vdim + PAD)) * 2; }
static size_t out_smem(int dim, int vcols) {                  // vcols: the value columns of one CTA
    return (size_t)C * (2 * (dim + PAD) + (vcols + PAD)) * 2 + (size_t)2 * dim * (vcols + PAD) * 2 + (size_t)C * (C + PAD) * 2 +
           (size_t)(THREADS / 32) * 16 * 20 * 4;
}
}  // namespace lt

}  // namespace imparo

using namespace imparo;

// q, k, v: pointers to the first row's q / k / v stretch (heads*dim, heads*dim, heads*vdim wide) inside rows of
// row_stride elements.  state: float [n_slots, heads, dim, vdim].  out: float [n_tok, heads*vdim].
extern "C" int imparo_linear_attention_recurrent(const void* q, const void* k, const void* v, long long row_stride, int dtype,
                                                 int act_silu, const float* decay, float* state, const int* item_row_start,
                                                 const int* item_slot, int n_items, int n_slots, float* out, int heads, int dim,
                                                 int vdim, int* status, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (dim < 1 || dim > 256 || vdim < 1 || heads < 1 || heads > 65535) return -3;
    dim3 grid(n_items, heads, (vdim + 31) / 32);
#define IMPARO_LA3(T_, D_, S_) launch(linear_attention_recurrent_kernel<T_, D_, S_>, grid, dim3(32), 0, stream, (const T_*)q, (const T_*)k, \
        (const T_*)v, (size_t)row_stride, decay, state, item_row_start, item_slot, n_slots, out, heads, dim, vdim, status)
#define IMPARO_LA2(T_, D_) do { if (act_silu) IMPARO_LA3(T_, D_, true); else IMPARO_LA3(T_, D_, false); } while (0)
#define IMPARO_LA(T_) do { if (dim <= 32) IMPARO_LA2(T_, 32); else if (dim <= 64) IMPARO_LA2(T_, 64); \
                           else if (dim <= 128) IMPARO_LA2(T_, 128); else IMPARO_LA2(T_, 256); } while (0)
    if (dtype == IMPARO_DT_F32) IMPARO_LA(float);
    else if (dtype == IMPARO_DT_BF16) IMPARO_LA(__nv_bfloat16);
    else return -1;
#undef IMPARO_LA
#undef IMPARO_LA2
#undef IMPARO_LA3
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// The same for batches with long portions: chunk rows per chunk, chunk_state: float scratch
// [rows / chunk + requests, heads, dim, vdim] (an upper bound of the number of chunks).
extern "C" int imparo_linear_attention_chunked(const void* q, const void* k, const void* v, long long row_stride, int dtype,
                                               int act_silu, const float* decay, float* state, float* chunk_state, int chunk,
                                               int max_chunks, const int* item_row_start, const int* item_slot, int n_items,
                                               int n_slots, float* out, int heads, int dim, int vdim, int* status,
                                               cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (dim < 1 || dim > 256 || vdim < 1 || heads < 1 || heads > 65535 || chunk < 1 || max_chunks < 1) return -3;
    const bool tensor = dtype == IMPARO_DT_BF16 && chunk == lt::C && dim % 16 == 0 && vdim % 16 == 0 && dim <= 128 && vdim <= 128 &&
                        row_stride % 8 == 0 && (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0 && (heads * dim) % 8 == 0;
    if (tensor) {
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaSuccess;
            const int most_out = (int)lt::out_smem(128, 128), most_local = (int)lt::local_smem(128, 128);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(lt::local_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most_local);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(lt::local_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most_local);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(lt::out_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most_out);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(lt::out_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most_out);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
        const lt::bf16 *qb = (const lt::bf16*)q, *kb = (const lt::bf16*)k, *vb = (const lt::bf16*)v;
        dim3 tgrid(max_chunks, heads);
        if (act_silu) launch(lt::local_kernel<true>, tgrid, dim3(lt::THREADS), lt::local_smem(dim, vdim), stream, kb, vb, (size_t)row_stride,
                             decay, chunk_state, item_row_start, n_items, heads, dim, vdim);
        else launch(lt::local_kernel<false>, tgrid, dim3(lt::THREADS), lt::local_smem(dim, vdim), stream, kb, vb, (size_t)row_stride,
                    decay, chunk_state, item_row_start, n_items, heads, dim, vdim);
        IMPARO_CHECK_LAUNCH();
        const int per_head_t = dim * vdim;
        launch(linear_attention_scan_kernel, dim3(n_items, heads, (per_head_t + 255) / 256), dim3(256), 0, stream, decay, chunk_state, state,
               item_row_start, item_slot, n_items, n_slots, chunk, heads, per_head_t, status);
        IMPARO_CHECK_LAUNCH();
        // two CTAs per (chunk, head), half of the value columns each, when a half is still whole tiles with 16-byte rows
        const int zsplit = (vdim >= 64 && vdim % 32 == 0) ? 2 : 1;
        dim3 ogrid(max_chunks, heads, zsplit);
        const size_t osmem = lt::out_smem(dim, vdim / zsplit);
        if (act_silu) launch(lt::out_kernel<true>, ogrid, dim3(lt::THREADS), osmem, stream, qb, kb, vb, (size_t)row_stride,
                             decay, (const float*)chunk_state, item_row_start, n_items, out, heads, dim, vdim);
        else launch(lt::out_kernel<false>, ogrid, dim3(lt::THREADS), osmem, stream, qb, kb, vb, (size_t)row_stride,
                    decay, (const float*)chunk_state, item_row_start, n_items, out, heads, dim, vdim);
        IMPARO_CHECK_LAUNCH();
        return 0;
    }
    dim3 grid(max_chunks, heads, (vdim + 31) / 32);
#define IMPARO_LC4(T_, D_, S_, O_) launch(linear_attention_chunk_kernel<T_, D_, S_, O_>, grid, dim3(32), 0, stream, (const T_*)q, \
        (const T_*)k, (const T_*)v, (size_t)row_stride, decay, chunk_state, item_row_start, n_items, chunk, out, heads, dim, vdim)
#define IMPARO_LC3(T_, D_, O_) do { if (act_silu) IMPARO_LC4(T_, D_, true, O_); else IMPARO_LC4(T_, D_, false, O_); } while (0)
#define IMPARO_LC2(T_, O_) do { if (dim <= 32) IMPARO_LC3(T_, 32, O_); else if (dim <= 64) IMPARO_LC3(T_, 64, O_); \
                                else if (dim <= 128) IMPARO_LC3(T_, 128, O_); else IMPARO_LC3(T_, 256, O_); } while (0)
#define IMPARO_LC(O_) do { if (dtype == IMPARO_DT_F32) IMPARO_LC2(float, O_); else if (dtype == IMPARO_DT_BF16) IMPARO_LC2(__nv_bfloat16, O_); \
                           else return -1; } while (0)
    IMPARO_LC(false);
    IMPARO_CHECK_LAUNCH();
    const int per_head = dim * vdim;
    launch(linear_attention_scan_kernel, dim3(n_items, heads, (per_head + 255) / 256), dim3(256), 0, stream, decay, chunk_state, state,
           item_row_start, item_slot, n_items, n_slots, chunk, heads, per_head, status);
    IMPARO_CHECK_LAUNCH();
    IMPARO_LC(true);
    IMPARO_CHECK_LAUNCH();
#undef IMPARO_LC
#undef IMPARO_LC2
#undef IMPARO_LC3
#undef IMPARO_LC4
    return 0;
}
