// A gated linear recurrence with a matrix state per head (the HGRN2 form of linear attention):
//
//     S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T          S: [dim, vdim] per head, float32
//     o_t = S_t^T q_t
//
// with q = silu(zq), f = low + (1 - low) * sigmoid(zf + bias): the forget gate also decides what is
// written, there is no key.  The state lives in a per-slot area of the cache, starts at zero when a
// slot is handed out and is carried from step to step, so a prompt may be cut anywhere and a decode
// step is the same kernels with one token per sequence.  Everything here is float32: gates,
// sigmoid, the state, the per-head RMS norm that follows.
//
// Three kernels, all reading the step's arrays on the device (graph-safe):
//   prepare  zq <- silu(zq), zf <- low + (1 - low) sigmoid(zf + bias), in place, every token at once
//   scan     per (sequence, head, tile of value columns): the recurrence over the sequence's new
//            tokens in order; o_t overwrites v_t in place; the state is read first and written last
//   norm     per (token, head): o / sqrt(mean(o^2) + eps) * w * out_scale -> the run dtype
//
// The projections z = [zq | zf | v] arrive as one float32 matrix [tokens, ld].
#include "common.cuh"

using namespace ri;

namespace {

__device__ __forceinline__ float sigmoid_f32(float x) {
    if (x >= 0.f) return 1.f / (1.f + expf(-x));
    const float e = expf(x);
    return e / (1.f + e);
}

__global__ void recurrence_prepare_kernel(float* __restrict__ z, int ld, const float* __restrict__ bias,
                                          const float* __restrict__ low, int n_tokens, int qdim) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    const size_t total = (size_t)n_tokens * qdim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / qdim), c = (int)(i % qdim);
        float* row = z + (size_t)t * ld;
        row[c] = silu_f32(row[c]);
        const float l = low[c];
        row[qdim + c] = l + (1.f - l) * sigmoid_f32(row[qdim + c] + bias[c]);
    }
}

// Threads of a warp: lane = column_in_warp * R + r.  Thread (r, j) keeps the rows r, r + R, r + 2R, ...
// of column j of the state in registers; the sum over rows of S[i, j] q[i] is finished by log2(R)
// shuffles inside the warp.  No block-wide barrier in the loop.
constexpr int R = 8;                 // row slices per column
constexpr int COLS = 32;             // value columns per block
constexpr int SCAN_THREADS = R * COLS;

template <int ROWS>
__global__ void __launch_bounds__(SCAN_THREADS)
recurrence_scan_kernel(float* __restrict__ z, int ld, float* __restrict__ state, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ seq_slot, int heads, int dim, int vdim) {
    const int b = blockIdx.x, h = blockIdx.y;
    const int r = threadIdx.x % R;
    const int j = blockIdx.z * COLS + threadIdx.x / R;
    const bool live = j < vdim;
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    const int slot = seq_slot[b];
    if (!RI_BLOCK_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT)) return;
    float* S = state + (((size_t)slot * heads + h) * dim) * vdim;
    float s[ROWS];
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
        const int i = r + k * R;
        s[k] = (live && i < dim) ? S[(size_t)i * vdim + j] : 0.f;
    }
    const int qdim = heads * dim;
    for (int t = t0; t < t1; ++t) {
        float* row = z + (size_t)t * ld;
        const float* q = row + h * dim;
        const float* f = row + qdim + h * dim;
        const float v = live ? row[2 * qdim + h * vdim + j] : 0.f;
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < ROWS; ++k) {
            const int i = r + k * R;
            if (i < dim) {
                const float fi = f[i];
                s[k] = fmaf(fi, s[k], (1.f - fi) * v);
                acc = fmaf(s[k], q[i], acc);
            }
        }
#pragma unroll
        for (int o = R / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (live && r == 0) row[2 * qdim + h * vdim + j] = acc;       // every lane of this column has read v
    }
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
        const int i = r + k * R;
        if (live && i < dim) S[(size_t)i * vdim + j] = s[k];
    }
}

// One warp per (token, head): RMS norm over the head's vdim values with one weight shared by heads.
template <typename T>
__global__ void headwise_rmsnorm_kernel(const float* __restrict__ x, int ld, int col0, const float* __restrict__ w,
                                        T* __restrict__ out, int out_ld, int n_tokens, int heads, int vdim,
                                        float eps, float out_scale) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_tokens * heads) return;
    const int t = warp / heads, h = warp % heads;
    const float* src = x + (size_t)t * ld + col0 + h * vdim;
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) ss = fmaf(src[d], src[d], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    T* dst = out + (size_t)t * out_ld + h * vdim;
    for (int d = lane; d < vdim; d += 32) dst[d] = from_f32<T>(src[d] * inv * w[d] * out_scale);
}

}  // namespace

// z: float32 [n_tokens, ld] = [zq (heads*dim) | zf (heads*dim) | v (heads*vdim)], overwritten.
// state: float32 [slots, heads, dim, vdim].  out: [n_tokens, heads*vdim] in `dtype`.
RI_API int ri_gated_recurrence(float* z, int ld, const float* bias, const float* low, const float* norm_w,
                               float* state, const int* cu_seqlens, const int* seq_slot, void* out, int dtype,
                               int n_tokens, int n_seqs, int heads, int dim, int vdim, float eps, float out_scale,
                               cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (ld < 2 * heads * dim + heads * vdim) return fail("gated_recurrence: rows of %d values are too short", ld);
    if (heads > 65535) return fail("gated_recurrence: %d heads exceed the grid limit", heads);
    const int rows = (dim + R - 1) / R;
    if (rows > 64) return fail("gated_recurrence: a head of %d channels exceeds %d", dim, 64 * R);
    const int qdim = heads * dim;
    {
        const size_t total = (size_t)n_tokens * qdim;
        const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
        cudaError_t e = launch_dependent(recurrence_prepare_kernel, blocks, 256, 0, stream, z, ld, bias, low, n_tokens, qdim);
        if (check_launch(e, "gated_recurrence (prepare)")) return 1;
    }
    {
        dim3 grid(n_seqs, heads, (vdim + COLS - 1) / COLS);
        cudaError_t e;
        if (rows <= 8)
            e = launch_dependent(recurrence_scan_kernel<8>, grid, SCAN_THREADS, 0, stream, z, ld, state, cu_seqlens, seq_slot, heads, dim, vdim);
        else if (rows <= 16)
            e = launch_dependent(recurrence_scan_kernel<16>, grid, SCAN_THREADS, 0, stream, z, ld, state, cu_seqlens, seq_slot, heads, dim, vdim);
        else if (rows <= 32)
            e = launch_dependent(recurrence_scan_kernel<32>, grid, SCAN_THREADS, 0, stream, z, ld, state, cu_seqlens, seq_slot, heads, dim, vdim);
        else
            e = launch_dependent(recurrence_scan_kernel<64>, grid, SCAN_THREADS, 0, stream, z, ld, state, cu_seqlens, seq_slot, heads, dim, vdim);
        if (check_launch(e, "gated_recurrence (scan)")) return 1;
    }
    {
        const long long warps = (long long)n_tokens * heads;
        const int blocks = (int)((warps * 32 + 255) / 256);
        cudaError_t e;
        if (dtype == RI_F32)
            e = launch_dependent(headwise_rmsnorm_kernel<float>, blocks, 256, 0, stream, (const float*)z, ld, 2 * qdim, norm_w,
                                 (float*)out, heads * vdim, n_tokens, heads, vdim, eps, out_scale);
        else if (dtype == RI_BF16)
            e = launch_dependent(headwise_rmsnorm_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const float*)z, ld, 2 * qdim,
                                 norm_w, (__nv_bfloat16*)out, heads * vdim, n_tokens, heads, vdim, eps, out_scale);
        else
            return fail("gated_recurrence: unknown dtype %d", dtype);
        return check_launch(e, "gated_recurrence (norm)");
    }
}

RI_DEFINE_LAST_ERROR()
