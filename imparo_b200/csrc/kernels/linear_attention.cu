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
    int c = first;
    for (int r = r0; r < r1; r += chunk, ++c) {
        const int n = min(chunk, r1 - r);
        float* cp = chunk_state + ((size_t)c * heads + h) * per_head + e;
        const float local = *cp;
        *cp = s;
        s = (n == chunk ? dec_full : powf(dec, (float)n)) * s + local;
    }
    *sp = s;
}

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
