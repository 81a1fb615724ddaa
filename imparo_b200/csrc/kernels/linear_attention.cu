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

template <typename T, int DMAX, bool SILU>
__global__ void __launch_bounds__(32)
linear_attention_recurrent_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, size_t row_stride,
                                  const float* __restrict__ decay, float* __restrict__ state,
                                  const int* __restrict__ item_row_start, const int* __restrict__ item_slot, int n_slots,
                                  float* __restrict__ out, int heads, int dim, int vdim, int* status) {
    __shared__ float qs[LA_STAGE][DMAX], ks[LA_STAGE][DMAX], vs[LA_STAGE][32];
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
    for (int base = r0; base < r1; base += LA_STAGE) {
        const int n = min(LA_STAGE, r1 - base);
        __syncwarp();
        for (int r = 0; r < n; ++r) {
            const T* qr = q + (size_t)(base + r) * row_stride + (size_t)h * dim;
            const T* kr = k + (size_t)(base + r) * row_stride + (size_t)h * dim;
            for (int d = lane; d < DMAX; d += 32) {
                float a = 0.f, b = 0.f;
                if (d < dim) {
                    a = to_f32(qr[d]); b = to_f32(kr[d]);
                    if (SILU) { a = silu(a); b = silu(b); }
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
            if (live) out[(size_t)(base + r) * ((size_t)heads * vdim) + (size_t)h * vdim + col] = o;
        }
    }
    if (live) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d) if (d < dim) sp[(size_t)d * vdim] = S[d];
    }
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
