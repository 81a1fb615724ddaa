// The selective state-space mixer (Mamba-2 form) over ragged batches, state in the request's slot.
//
// One projection row holds [z: inner | x: inner | B: groups*N | C: groups*N | dt: heads], inner = heads * vdim.
//  (1) mamba2_conv: causal convolution per channel over [x | B | C] with a bias, then silu; inputs before a
//      portion's first row come from the slot's conv state (the last taps-1 inputs, oldest first), zeros for a
//      fresh request (the slot is cleared).  The same launch makes the step sizes dt = softplus(dt + dt_bias) in
//      32-bit.  A second small kernel then moves the conv state on (it runs after every reader of the old state).
//  (2) mamba2_scan: per request, head and 32 value columns one to four warps walk the rows in order with the state column
//      S[:, p] in their registers (a stretch each):  S = exp(-exp(A_log) dt) S + dt B x[p];  y[p] = C . S + D x[p].  Decays, step sizes
//      and the state are 32-bit in both precisions.
//  (3) Long portions run in chunks of L rows side by side (three launches, as the decayed linear attention does):
//      every chunk's own state from zero and its total decay (as a product of weighted B rows with x rows for states up
//      to 128, else by walking the rows); a scan over each request's chunks that leaves every
//      chunk's starting state and the request's new state; every chunk's outputs from its starting state plus the
//      rows inside the chunk.  32-bit on CUDA cores.
//  (4) gate_group_rmsnorm: y * silu(z), then an RMS norm over each of `groups` equal stretches of the row, times a
//      weight.
#include "common.cuh"

namespace imparo {

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---- (1) convolution + step sizes ------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
mamba2_conv_kernel(const T* __restrict__ proj, size_t stride, int x_off, int dt_off, int channels, int heads, int taps,
                   const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ dt_bias,
                   const float* __restrict__ state, const int* __restrict__ item_row_start,
                   const int* __restrict__ item_of_token, const int* __restrict__ item_slot, int n_slots,
                   float* __restrict__ xbc, float* __restrict__ dt, int* status) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int item = item_of_token[t];
    const int first = item_row_start[item];
    const int slot = item_slot[item];
    pdl_wait();
    if (c >= channels + heads) return;
    if (c >= channels) {                                          // a step size
        const int h = c - channels;
        dt[(size_t)t * heads + h] = softplus_f(to_f32(proj[(size_t)t * stride + dt_off + h]) + dt_bias[h]);
        return;
    }
    if (slot < 0 || slot >= n_slots) {
        if (c == 0) report(status, IMPARO_ST_SLOT_RANGE, 61, t, slot);
        return;
    }
    const float* st = state + (size_t)slot * (taps - 1) * channels;
    float acc = bias ? bias[c] : 0.f;
    const int j = t - first;                                      // row within the portion
    for (int k = 0; k < taps; ++k) {
        const int src = j - (taps - 1 - k);
        const float u = src >= 0 ? to_f32(proj[(size_t)(first + src) * stride + x_off + c])
                                 : st[(size_t)(taps - 1 + src) * channels + c];
        acc += w[(size_t)c * taps + k] * u;
    }
    xbc[(size_t)t * channels + c] = silu(acc);
}

template <typename T>
__global__ void __launch_bounds__(256)
mamba2_conv_state_kernel(const T* __restrict__ proj, size_t stride, int x_off, int channels, int taps,
                         float* __restrict__ state, const int* __restrict__ item_row_start,
                         const int* __restrict__ item_slot, int n_slots) {
    pdl_trigger();
    const int item = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int first = item_row_start[item], n = item_row_start[item + 1] - first;
    const int slot = item_slot[item];
    pdl_wait();
    if (c >= channels || slot < 0 || slot >= n_slots) return;
    float* st = state + (size_t)slot * (taps - 1) * channels;
    const int keep = taps - 1;
    // entry i of the new state is input number (n - keep + i) of the portion; negative numbers are old entries
    float moved[16];
    for (int i = 0; i < keep; ++i) {
        const int src = n - keep + i;
        moved[i] = src >= 0 ? to_f32(proj[(size_t)(first + src) * stride + x_off + c]) : st[(size_t)(keep + src) * channels + c];
    }
    for (int i = 0; i < keep; ++i) st[(size_t)i * channels + c] = moved[i];
}

// ---- (2) the recurrence, row by row ------------------------------------------------------------------------------
// One row of the recurrence for this thread's state column: S = decay S + dx B;  returns C . S.  B and C come from shared
// memory four at a time; entries from N on are zero there and in S, so the loops run over the whole NMAX.  Four partial
// sums (two packed pairs) keep the additions from waiting on one another; their order is fixed.
template <int NMAX>
__device__ __forceinline__ float state_step(float (&S)[NMAX], const float* __restrict__ b, const float* __restrict__ c, float decay, float dx) {
    // two 32-bit operations per instruction (fma.rn.f32x2): each half rounds as the single operation does
    const float2 d2 = make_float2(decay, decay), x2 = make_float2(dx, dx);
    float2 a01 = make_float2(0.f, 0.f), a23 = make_float2(0.f, 0.f);
#pragma unroll
    for (int n = 0; n < NMAX; n += 4) {
        const float4 b4 = *reinterpret_cast<const float4*>(b + n);
        const float4 c4 = *reinterpret_cast<const float4*>(c + n);
        float2 s01 = make_float2(S[n], S[n + 1]), s23 = make_float2(S[n + 2], S[n + 3]);
        s01 = __ffma2_rn(d2, s01, __fmul2_rn(make_float2(b4.x, b4.y), x2));
        s23 = __ffma2_rn(d2, s23, __fmul2_rn(make_float2(b4.z, b4.w), x2));
        a01 = __ffma2_rn(s01, make_float2(c4.x, c4.y), a01);
        a23 = __ffma2_rn(s23, make_float2(c4.z, c4.w), a23);
        S[n] = s01.x; S[n + 1] = s01.y; S[n + 2] = s23.x; S[n + 3] = s23.y;
    }
    return (a01.x + a01.y) + (a23.x + a23.y);
}

template <int NMAX>
__device__ __forceinline__ void state_step_no_out(float (&S)[NMAX], const float* __restrict__ b, float decay, float dx) {
    const float2 d2 = make_float2(decay, decay), x2 = make_float2(dx, dx);
#pragma unroll
    for (int n = 0; n < NMAX; n += 4) {
        const float4 b4 = *reinterpret_cast<const float4*>(b + n);
        float2 s01 = make_float2(S[n], S[n + 1]), s23 = make_float2(S[n + 2], S[n + 3]);
        s01 = __ffma2_rn(d2, s01, __fmul2_rn(make_float2(b4.x, b4.y), x2));
        s23 = __ffma2_rn(d2, s23, __fmul2_rn(make_float2(b4.z, b4.w), x2));
        S[n] = s01.x; S[n + 1] = s01.y; S[n + 2] = s23.x; S[n + 3] = s23.y;
    }
}

// A row's B and C entries of this lane within its warp's share of the state (n = n0 + lane, n0 + lane + 32, ...), its step
// size and its x value, fetched ahead of the row being computed (the kernels keep two rows in flight), so that their latency
// hides behind the arithmetic.
template <int NH>
struct RowAhead {
    static constexpr int PER = (NH + 31) / 32;
    float b[PER], c[PER], step, x;
    __device__ __forceinline__ void fetch(const float* __restrict__ xbc, const float* __restrict__ dt, int t, int channels,
                                          int b_off, int c_off, int x_col, int heads, int h, int n0, int N, int lane, bool live,
                                          bool want_c) {
        const float* row = xbc + (size_t)t * channels;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int n = n0 + lane + 32 * i;
            const bool in = lane + 32 * i < NH && n < N;
            b[i] = in ? row[b_off + n] : 0.f;
            c[i] = (want_c && in) ? row[c_off + n] : 0.f;
        }
        step = dt[(size_t)t * heads + h];
        x = live ? row[x_col] : 0.f;
    }
    __device__ __forceinline__ void put(float* __restrict__ bs, float* __restrict__ cs, int lane) const {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int n = lane + 32 * i;
            if (n < NH) { bs[n] = b[i]; if (cs) cs[n] = c[i]; }
        }
    }
};

// The state column S[:, p] of a (request, head, value column) is cut into SPLIT stretches of NH entries, one warp each
// (fewer registers per thread, more warps per SM); the warps' shares of C . S meet in shared memory, added in warp order.
// grid (heads, items, ceil(vdim / 32)), SPLIT warps
template <int NH, int SPLIT>
__global__ void __launch_bounds__(32 * SPLIT, SPLIT == 1 ? 16 : (SPLIT == 2 ? 8 : 4))
mamba2_scan_kernel(const float* __restrict__ xbc, const float* __restrict__ dt, const float* __restrict__ A_log,
                   const float* __restrict__ D, float* __restrict__ state, const int* __restrict__ item_row_start,
                   const int* __restrict__ item_slot, int n_slots, float* __restrict__ y,
                   int heads, int vdim, int N, int groups, int* status) {
    __shared__ __align__(16) float bc[SPLIT][2][NH];
    __shared__ float part[2][SPLIT][32];
    pdl_trigger();
    const int h = blockIdx.x, item = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = blockIdx.z * 32 + lane;
    const int first = item_row_start[item], last = item_row_start[item + 1];
    const int slot = item_slot[item];
    const float a = -expf(A_log[h]);
    const float d_skip = D[h];
    pdl_wait();
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0 && blockIdx.z == 0 && h == 0) report(status, IMPARO_ST_SLOT_RANGE, 62, item, slot);
        return;
    }
    const int inner = heads * vdim, channels = inner + 2 * groups * N;
    const int g = h / (heads / groups);
    const bool live = p < vdim;
    const int n0 = warp * NH;
    float* sp = state + (((size_t)slot * heads + h) * N) * vdim + p;
    float S[NH];
#pragma unroll
    for (int n = 0; n < NH; ++n) S[n] = (live && n0 + n < N) ? sp[(size_t)(n0 + n) * vdim] : 0.f;
    RowAhead<NH> next, after;                          // the rows one and two ahead of the one being computed
    const int b_off = inner + g * N, c_off = inner + groups * N + g * N, x_col = h * vdim + p;
    if (first < last) next.fetch(xbc, dt, first, channels, b_off, c_off, x_col, heads, h, n0, N, lane, live, true);
    if (first + 1 < last) after.fetch(xbc, dt, first + 1, channels, b_off, c_off, x_col, heads, h, n0, N, lane, live, true);
    for (int t = first; t < last; ++t) {
        __syncwarp();
        next.put(bc[warp][0], bc[warp][1], lane);
        __syncwarp();
        const float step = next.step, xv = next.x;
        next = after;
        if (t + 2 < last) after.fetch(xbc, dt, t + 2, channels, b_off, c_off, x_col, heads, h, n0, N, lane, live, true);
        float acc = state_step<NH>(S, bc[warp][0], bc[warp][1], expf(a * step), step * xv);
        if (SPLIT > 1) {
            const int buf = (t - first) & 1;
            part[buf][warp][lane] = acc;
            __syncthreads();
            acc = part[buf][0][lane];
#pragma unroll
            for (int w = 1; w < SPLIT; ++w) acc += part[buf][w][lane];
        }
        if (warp == 0 && live) y[(size_t)t * inner + h * vdim + p] = acc + d_skip * xv;
    }
    if (live) {
#pragma unroll
        for (int n = 0; n < NH; ++n)
            if (n0 + n < N) sp[(size_t)(n0 + n) * vdim] = S[n];
    }
}

// ---- (3) long portions in chunks -----------------------------------------------------------------------------------
// Chunk c of the launch covers rows [lo, hi) of one request (chunks never straddle requests): chunk_item[c],
// chunk_lo[c], chunk_hi[c] are made by a small kernel from item_row_start.  Unused chunks have lo == hi.
__global__ void mamba2_chunk_plan_kernel(const int* __restrict__ item_row_start, int n_items, int L, int max_chunks,
                                         int* __restrict__ chunk_item, int* __restrict__ chunk_lo, int* __restrict__ chunk_hi,
                                         int* __restrict__ item_chunk_start) {
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int c = 0;
    for (int i = 0; i < n_items; ++i) {
        item_chunk_start[i] = c;
        for (int lo = item_row_start[i]; lo < item_row_start[i + 1] && c < max_chunks; lo += L) {
            chunk_item[c] = i; chunk_lo[c] = lo; chunk_hi[c] = min(lo + L, item_row_start[i + 1]);
            ++c;
        }
    }
    item_chunk_start[n_items] = c;
    for (; c < max_chunks; ++c) { chunk_item[c] = -1; chunk_lo[c] = 0; chunk_hi[c] = 0; }
}

// every chunk's own state from zero [chunk, heads, N, vdim] and the chunk's total decay [chunk, heads]
template <int NH, int SPLIT>
__global__ void __launch_bounds__(32 * SPLIT, SPLIT == 1 ? 16 : (SPLIT == 2 ? 8 : 4))
mamba2_chunk_state_kernel(const float* __restrict__ xbc, const float* __restrict__ dt, const float* __restrict__ A_log,
                          const int* __restrict__ chunk_lo, const int* __restrict__ chunk_hi,
                          float* __restrict__ chunk_state, float* __restrict__ chunk_decay,
                          int heads, int vdim, int N, int groups) {
    __shared__ __align__(16) float bs[SPLIT][NH];
    pdl_trigger();
    const int h = blockIdx.x, c = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = blockIdx.z * 32 + lane;
    const float a = -expf(A_log[h]);
    pdl_wait();
    const int lo = chunk_lo[c], hi = chunk_hi[c];
    if (lo >= hi) return;
    const int inner = heads * vdim, channels = inner + 2 * groups * N;
    const int g = h / (heads / groups);
    const bool live = p < vdim;
    const int n0 = warp * NH;
    float S[NH];
#pragma unroll
    for (int n = 0; n < NH; ++n) S[n] = 0.f;
    float total = 0.f;                                            // sum of a * dt over the chunk
    RowAhead<NH> next, after;
    const int b_off = inner + g * N, x_col = h * vdim + p;
    next.fetch(xbc, dt, lo, channels, b_off, 0, x_col, heads, h, n0, N, lane, live, false);
    if (lo + 1 < hi) after.fetch(xbc, dt, lo + 1, channels, b_off, 0, x_col, heads, h, n0, N, lane, live, false);
    for (int t = lo; t < hi; ++t) {
        __syncwarp();
        next.put(bs[warp], nullptr, lane);
        __syncwarp();
        const float step = next.step, xv = next.x;
        next = after;
        if (t + 2 < hi) after.fetch(xbc, dt, t + 2, channels, b_off, 0, x_col, heads, h, n0, N, lane, live, false);
        total += a * step;
        state_step_no_out<NH>(S, bs[warp], expf(a * step), step * xv);
    }
    if (live) {
        float* out = chunk_state + (((size_t)c * heads + h) * N) * vdim + p;
#pragma unroll
        for (int n = 0; n < NH; ++n)
            if (n0 + n < N) out[(size_t)(n0 + n) * vdim] = S[n];
    }
    if (threadIdx.x == 0 && blockIdx.z == 0) chunk_decay[(size_t)c * heads + h] = total;
}

// The same as a product, for state sizes up to 128 and chunks of up to 64 rows: with w_t = dt_t exp(sum over the rows r
// after t of a dt_r), the chunk's own state is S[n, p] = sum_t (w_t B_t[n]) x_t[p].  A block per (head, chunk, 32 value
// columns): the weighted B rows and the x rows in shared memory, every thread a patch of 4 x 4 of S, rows added in order.
// grid (heads, chunks, ceil(vdim / 32)), 256 threads
constexpr int SM_L = 64, SM_N = 128, SM_P = 32;
__global__ void __launch_bounds__(256)
mamba2_chunk_state_mm_kernel(const float* __restrict__ xbc, const float* __restrict__ dt, const float* __restrict__ A_log,
                             const int* __restrict__ chunk_lo, const int* __restrict__ chunk_hi,
                             float* __restrict__ chunk_state, float* __restrict__ chunk_decay,
                             int heads, int vdim, int N, int groups) {
    __shared__ __align__(16) float bw[SM_L][SM_N];
    __shared__ __align__(16) float xs[SM_L][SM_P];
    __shared__ float adt[SM_L], wt[SM_L];
    pdl_trigger();
    const int h = blockIdx.x, c = blockIdx.y, p0 = blockIdx.z * SM_P, tid = threadIdx.x;
    const float a = -expf(A_log[h]);
    pdl_wait();
    const int lo = chunk_lo[c], hi = chunk_hi[c];
    if (lo >= hi) return;
    const int len = hi - lo;
    const int inner = heads * vdim, channels = inner + 2 * groups * N;
    const int g = h / (heads / groups);
    if (tid < SM_L) adt[tid] = tid < len ? a * dt[(size_t)(lo + tid) * heads + h] : 0.f;
    __syncthreads();
    if (tid < SM_L) {
        float after = 0.f;                                        // sum of a dt over the rows after this one, last row first
        for (int r = len - 1; r > tid; --r) after += adt[r];
        wt[tid] = tid < len ? dt[(size_t)(lo + tid) * heads + h] * expf(after) : 0.f;
        if (tid == 0 && blockIdx.z == 0) chunk_decay[(size_t)c * heads + h] = after + adt[0];
    }
    __syncthreads();
    for (int i = tid; i < SM_L * SM_N; i += 256) {
        const int t = i / SM_N, n = i - t * SM_N;
        bw[t][n] = (t < len && n < N) ? wt[t] * xbc[(size_t)(lo + t) * channels + inner + g * N + n] : 0.f;
    }
    for (int i = tid; i < SM_L * SM_P; i += 256) {
        const int t = i / SM_P, pp = i - t * SM_P;
        xs[t][pp] = (t < len && p0 + pp < vdim) ? xbc[(size_t)(lo + t) * channels + h * vdim + p0 + pp] : 0.f;
    }
    __syncthreads();
    const int tn = (tid >> 3) * 4, tp = (tid & 7) * 4;             // 32 x 8 threads, a patch of 4 state entries x 4 columns each
    float acc[4][4] = {};
    for (int t = 0; t < len; ++t) {
        const float4 b4 = *reinterpret_cast<const float4*>(&bw[t][tn]);
        const float4 x4 = *reinterpret_cast<const float4*>(&xs[t][tp]);
        const float bv[4] = {b4.x, b4.y, b4.z, b4.w}, xv[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(bv[i], xv[j], acc[i][j]);
    }
    float* out = chunk_state + (((size_t)c * heads + h) * N) * vdim;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (tn + i < N && p0 + tp + j < vdim) out[(size_t)(tn + i) * vdim + p0 + tp + j] = acc[i][j];
}

// per request and head: chunk_state[c] becomes the state BEFORE chunk c; the slot gets the state after the last chunk
__global__ void __launch_bounds__(256)
mamba2_chunk_scan_kernel(float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                         const int* __restrict__ item_chunk_start, const int* __restrict__ item_slot, int n_slots,
                         float* __restrict__ state, int heads, int vdim, int N, int* status) {
    pdl_trigger();
    const int h = blockIdx.x, item = blockIdx.y;
    const int slot = item_slot[item];
    pdl_wait();
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0 && h == 0 && blockIdx.z == 0) report(status, IMPARO_ST_SLOT_RANGE, 63, item, slot);
        return;
    }
    const int c0 = item_chunk_start[item], c1 = item_chunk_start[item + 1];
    const int per = N * vdim;
    for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < per; e += gridDim.z * blockDim.x) {
        float* sp = state + ((size_t)slot * heads + h) * per + e;
        float S = *sp;
        int c = c0;
        for (; c + 8 <= c1; c += 8) {                              // eight chunks' loads in flight
            float own[8], dec[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                own[u] = chunk_state[((size_t)(c + u) * heads + h) * per + e];
                dec[u] = expf(chunk_decay[(size_t)(c + u) * heads + h]);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                chunk_state[((size_t)(c + u) * heads + h) * per + e] = S;
                S = dec[u] * S + own[u];
            }
        }
        for (; c < c1; ++c) {
            float* cs = chunk_state + ((size_t)c * heads + h) * per + e;
            const float own = *cs;
            *cs = S;
            S = expf(chunk_decay[(size_t)c * heads + h]) * S + own;
        }
        *sp = S;
    }
}

// every chunk's outputs: the recurrence inside the chunk from its starting state (chunks side by side)
template <int NH, int SPLIT>
__global__ void __launch_bounds__(32 * SPLIT, SPLIT == 1 ? 16 : (SPLIT == 2 ? 8 : 4))
mamba2_chunk_out_kernel(const float* __restrict__ xbc, const float* __restrict__ dt, const float* __restrict__ A_log,
                        const float* __restrict__ D, const int* __restrict__ chunk_lo, const int* __restrict__ chunk_hi,
                        const float* __restrict__ chunk_state, float* __restrict__ y,
                        int heads, int vdim, int N, int groups) {
    __shared__ __align__(16) float bc[SPLIT][2][NH];
    __shared__ float part[2][SPLIT][32];
    pdl_trigger();
    const int h = blockIdx.x, c = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = blockIdx.z * 32 + lane;
    const float a = -expf(A_log[h]);
    const float d_skip = D[h];
    pdl_wait();
    const int lo = chunk_lo[c], hi = chunk_hi[c];
    if (lo >= hi) return;
    const int inner = heads * vdim, channels = inner + 2 * groups * N;
    const int g = h / (heads / groups);
    const bool live = p < vdim;
    const int n0 = warp * NH;
    const float* sp = chunk_state + (((size_t)c * heads + h) * N) * vdim + p;
    float S[NH];
#pragma unroll
    for (int n = 0; n < NH; ++n) S[n] = (live && n0 + n < N) ? sp[(size_t)(n0 + n) * vdim] : 0.f;
    RowAhead<NH> next, after;
    const int b_off = inner + g * N, c_off = inner + groups * N + g * N, x_col = h * vdim + p;
    next.fetch(xbc, dt, lo, channels, b_off, c_off, x_col, heads, h, n0, N, lane, live, true);
    if (lo + 1 < hi) after.fetch(xbc, dt, lo + 1, channels, b_off, c_off, x_col, heads, h, n0, N, lane, live, true);
    for (int t = lo; t < hi; ++t) {
        __syncwarp();
        next.put(bc[warp][0], bc[warp][1], lane);
        __syncwarp();
        const float step = next.step, xv = next.x;
        next = after;
        if (t + 2 < hi) after.fetch(xbc, dt, t + 2, channels, b_off, c_off, x_col, heads, h, n0, N, lane, live, true);
        float acc = state_step<NH>(S, bc[warp][0], bc[warp][1], expf(a * step), step * xv);
        if (SPLIT > 1) {
            const int buf = (t - lo) & 1;
            part[buf][warp][lane] = acc;
            __syncthreads();
            acc = part[buf][0][lane];
#pragma unroll
            for (int w = 1; w < SPLIT; ++w) acc += part[buf][w][lane];
        }
        if (warp == 0 && live) y[(size_t)t * inner + h * vdim + p] = acc + d_skip * xv;
    }
}

// ---- (4) gate, then a norm per stretch of the row ----------------------------------------------------------------
// grid (rows, groups): out[r, s] = (y silu(z))[r, s] / rms over the stretch * w[s]
template <typename T, typename TZ>
__global__ void __launch_bounds__(256)
gate_group_rmsnorm_kernel(const float* __restrict__ y, const TZ* __restrict__ z, size_t z_stride, const float* __restrict__ w,
                          float eps, T* __restrict__ out, int width, int groups) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, grp = blockIdx.y;
    const int per = width / groups;
    const float* yr = y + (size_t)r * width + (size_t)grp * per;
    const TZ* zr = z + (size_t)r * z_stride + (size_t)grp * per;
    float ss = 0.f;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const float v = yr[i] * silu(to_f32(zr[i]));
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)per + eps);
    T* o = out + (size_t)r * width + (size_t)grp * per;
    const float* wg = w + (size_t)grp * per;
    for (int i = threadIdx.x; i < per; i += blockDim.x)
        o[i] = from_f32<T>(yr[i] * silu(to_f32(zr[i])) * scale * wg[i]);
}

}  // namespace imparo

using namespace imparo;

// proj: [n_tok, >= dt_off + heads] rows of `stride` elements in dtype; xbc float32 [n_tok, channels]; dt float32
// [n_tok, heads]; state float32 [n_slots, taps-1, channels].  Two launches.
extern "C" int imparo_mamba2_conv(const void* proj, int dtype, long long stride, int x_off, int dt_off, int channels, int heads,
                                  int taps, const float* w, const float* bias, const float* dt_bias, float* state,
                                  const int* item_row_start, const int* item_of_token, const int* item_slot, int n_items,
                                  int n_slots, int n_tok, float* xbc, float* dt, int* status, cudaStream_t stream) {
    if (n_tok <= 0) return 0;
    if (taps < 1 || taps > 17) return -6;
    dim3 grid(n_tok, (channels + heads + 255) / 256), sgrid(n_items, (channels + 255) / 256);
    if (dtype == IMPARO_DT_F32) {
        launch(mamba2_conv_kernel<float>, grid, dim3(256), 0, stream, (const float*)proj, (size_t)stride, x_off, dt_off, channels, heads,
               taps, w, bias, dt_bias, (const float*)state, item_row_start, item_of_token, item_slot, n_slots, xbc, dt, status);
        IMPARO_CHECK_LAUNCH();
        if (taps > 1)
            launch(mamba2_conv_state_kernel<float>, sgrid, dim3(256), 0, stream, (const float*)proj, (size_t)stride, x_off, channels, taps,
                   state, item_row_start, item_slot, n_slots);
    } else if (dtype == IMPARO_DT_BF16) {
        launch(mamba2_conv_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)proj, (size_t)stride, x_off, dt_off,
               channels, heads, taps, w, bias, dt_bias, (const float*)state, item_row_start, item_of_token, item_slot, n_slots, xbc, dt,
               status);
        IMPARO_CHECK_LAUNCH();
        if (taps > 1)
            launch(mamba2_conv_state_kernel<__nv_bfloat16>, sgrid, dim3(256), 0, stream, (const __nv_bfloat16*)proj, (size_t)stride, x_off,
                   channels, taps, state, item_row_start, item_slot, n_slots);
    } else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// state entries per warp, warps per state column
#define MAMBA2_BY_N(CALL)                                       \
    do {                                                        \
        if (N <= 16) { CALL(16, 1); }                           \
        else if (N <= 32) { CALL(32, 1); }                      \
        else if (N <= 64) { CALL(32, 2); }                      \
        else if (N <= 128) { CALL(64, 2); }                     \
        else { CALL(64, 4); }                                   \
    } while (0)

extern "C" int imparo_mamba2_scan(const float* xbc, const float* dt, const float* A_log, const float* D, float* state,
                                  const int* item_row_start, const int* item_slot, int n_items, int n_slots, float* y,
                                  int heads, int vdim, int N, int groups, int* status, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (N < 1 || N > 256) return -3;
    if (groups < 1 || heads % groups) return -5;
    dim3 grid(heads, n_items, (vdim + 31) / 32);
#define CALL(NH, SP) launch(mamba2_scan_kernel<NH, SP>, grid, dim3(32 * SP), 0, stream, xbc, dt, A_log, D, state, item_row_start, \
                            item_slot, n_slots, y, heads, vdim, N, groups, status)
    MAMBA2_BY_N(CALL);
#undef CALL
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// scratch_i: int32 [3 * max_chunks + n_items + 1]; chunk_state float32 [max_chunks, heads, N, vdim]; chunk_decay float32
// [max_chunks, heads]; max_chunks >= n_tok / L + n_items.  Four launches.
extern "C" int imparo_mamba2_scan_chunked(const float* xbc, const float* dt, const float* A_log, const float* D, float* state,
                                          const int* item_row_start, const int* item_slot, int n_items, int n_slots, float* y,
                                          int heads, int vdim, int N, int groups, int L, int max_chunks, int* scratch_i,
                                          float* chunk_state, float* chunk_decay, int* status, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (N < 1 || N > 256) return -3;
    if (groups < 1 || heads % groups) return -5;
    if (L < 1 || max_chunks < 1) return -2;
    int* chunk_item = scratch_i;
    int* chunk_lo = scratch_i + max_chunks;
    int* chunk_hi = scratch_i + 2 * max_chunks;
    int* item_chunk_start = scratch_i + 3 * max_chunks;
    launch(mamba2_chunk_plan_kernel, dim3(1), dim3(32), 0, stream, item_row_start, n_items, L, max_chunks, chunk_item, chunk_lo,
           chunk_hi, item_chunk_start);
    IMPARO_CHECK_LAUNCH();
    dim3 grid(heads, max_chunks, (vdim + 31) / 32);
    if (N <= SM_N && L <= SM_L) {
        launch(mamba2_chunk_state_mm_kernel, grid, dim3(256), 0, stream, xbc, dt, A_log, (const int*)chunk_lo, (const int*)chunk_hi,
               chunk_state, chunk_decay, heads, vdim, N, groups);
    } else {
#define CALL(NH, SP) launch(mamba2_chunk_state_kernel<NH, SP>, grid, dim3(32 * SP), 0, stream, xbc, dt, A_log, (const int*)chunk_lo, \
                            (const int*)chunk_hi, chunk_state, chunk_decay, heads, vdim, N, groups)
        MAMBA2_BY_N(CALL);
#undef CALL
    }
    IMPARO_CHECK_LAUNCH();
    const int per = N * vdim;
    launch(mamba2_chunk_scan_kernel, dim3(heads, n_items, (per + 255) / 256), dim3(256), 0, stream, chunk_state,
           (const float*)chunk_decay, (const int*)item_chunk_start, item_slot, n_slots, state, heads, vdim, N, status);
    IMPARO_CHECK_LAUNCH();
#define CALL(NH, SP) launch(mamba2_chunk_out_kernel<NH, SP>, grid, dim3(32 * SP), 0, stream, xbc, dt, A_log, D, (const int*)chunk_lo, \
                            (const int*)chunk_hi, (const float*)chunk_state, y, heads, vdim, N, groups)
    MAMBA2_BY_N(CALL);
#undef CALL
    IMPARO_CHECK_LAUNCH();
    return 0;
}

// y float32 [rows, width]; z [rows, width] in rows of z_stride elements (z_dtype); out [rows, width] in out_dtype
extern "C" int imparo_gate_group_rmsnorm(const float* y, const void* z, int z_dtype, long long z_stride, const float* w, float eps,
                                         void* out, int out_dtype, int rows, int width, int groups, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (groups < 1 || width % groups) return -2;
    dim3 grid(rows, groups);
    if (z_dtype == IMPARO_DT_F32 && out_dtype == IMPARO_DT_F32)
        launch(gate_group_rmsnorm_kernel<float, float>, grid, dim3(256), 0, stream, y, (const float*)z, (size_t)z_stride, w, eps,
               (float*)out, width, groups);
    else if (z_dtype == IMPARO_DT_BF16 && out_dtype == IMPARO_DT_BF16)
        launch(gate_group_rmsnorm_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(256), 0, stream, y, (const __nv_bfloat16*)z,
               (size_t)z_stride, w, eps, (__nv_bfloat16*)out, width, groups);
    else if (z_dtype == IMPARO_DT_F32 && out_dtype == IMPARO_DT_BF16)
        launch(gate_group_rmsnorm_kernel<__nv_bfloat16, float>, grid, dim3(256), 0, stream, y, (const float*)z, (size_t)z_stride, w, eps,
               (__nv_bfloat16*)out, width, groups);
    else return -1;
    IMPARO_CHECK_LAUNCH();
    return 0;
}
