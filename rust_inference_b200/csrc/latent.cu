// Row-wise kernels of attention over a shared low-rank latent.
//
// Every position keeps one row of `rank` + `rd` values for all heads: the normalised latent c and one rotated
// key part.  A head's keys and values are linear maps of c (k_h = Uk_h c, v_h = Uv_h c), so its score against
// a cached position is q_nope . (Uk_h c) + q_rot . k_rot = (Uk_h^T q_nope) . c + q_rot . k_rot: with the query
// carried into the latent space the cached rows are the keys of ALL heads (one kv head whose key is the row
// and whose value is the row's first `rank` channels), and a head's output is Uv_h applied to the weighted
// sum of the latents.  The kernels here do what surrounds the products and the attention:
//
//   prepare    from the projection [T, ld] (q heads of d + rd channels, then rank + rd channels of the
//              latent with its rotated key part, if this layer writes them): RMS norm of the latent and
//              rotation of the key part into the cache row; the heads' unrotated query parts copied head by
//              head (a head's tokens consecutive: the rows of the per-head products), the rotated query
//              parts rotated into the wide query rows [T, heads, rank + rd]; and the lists that the grouped
//              products want (every head is a group of T rows).
//   widen      the per-head products' float32 results [heads, T, rank] into the wide query rows.
//   gate       out[t, h, :] = v[h, t, :] * sigmoid(g[t, h]): the heads' values (float32, head by head) times
//              the output gate, token by token, in the run dtype.
//
// Rotation, norm and sigmoid are float32.
#include "common.cuh"

using namespace ri;

namespace {

constexpr int PREPARE_HEADS = 4;    // query heads per block of the preparing kernel

// grid (tokens, groups of PREPARE_HEADS heads); the first group's block also writes the cache row and the lists
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                      const float* __restrict__ c_w, float eps, const int* __restrict__ token_pos,
                      const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                      const int* __restrict__ page_table, int max_pages, T* __restrict__ cache, T* __restrict__ q_nope,
                      T* __restrict__ q_wide, int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ tiles,
                      int* __restrict__ n_tiles, int n_tokens, int n_heads, int d, int rd, int rank, int rot, int style,
                      int page_size, int write_kv, int tile_rows, int vec) {
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    const int h0 = blockIdx.y * PREPARE_HEADS, nh = min(PREPARE_HEADS, n_heads - h0);
    const int pos = token_pos[t];                     // positions and tables: fixed before the step
    const int half = rot >> 1;
    const float* c = cos_t + (size_t)pos * half;
    const float* s = sin_t + (size_t)pos * half;
    let_next_kernel_start();
    wait_for_previous_kernels();                      // the projection; and the lists may still be read by the layer before
    const T* row = proj + (size_t)t * ld;
    const int qh = d + rd, wide = rank + rd;

    // queries: the unrotated parts head by head, the rotated parts into the wide rows
    if (vec) {                                        // 2-byte values, 16 bytes at a time
        const int d8 = d >> 3;
        for (int i = tid; i < nh * d8; i += blockDim.x) {
            const int h = h0 + i / d8, j = (i % d8) * 8;
            *reinterpret_cast<uint4*>(q_nope + ((size_t)h * n_tokens + t) * d + j) = *reinterpret_cast<const uint4*>(row + h * qh + j);
        }
    } else {
        for (int i = tid; i < nh * d; i += blockDim.x) {
            const int h = h0 + i / d, j = i % d;
            q_nope[((size_t)h * n_tokens + t) * d + j] = row[h * qh + j];
        }
    }
    for (int i = tid; i < nh * half; i += blockDim.x) {
        const int h = h0 + i / half, k = i % half;
        const int i0 = style == 0 ? k : 2 * k, i1 = style == 0 ? k + half : 2 * k + 1;
        const T* v = row + h * qh + d;
        const float x0 = to_f32<T>(v[i0]), x1 = to_f32<T>(v[i1]);
        T* dst = q_wide + ((size_t)t * n_heads + h) * wide + rank;
        dst[i0] = from_f32<T>(x0 * c[k] - x1 * s[k]);
        dst[i1] = from_f32<T>(x0 * s[k] + x1 * c[k]);
    }
    for (int i = tid; i < nh * (rd - rot); i += blockDim.x) {
        const int h = h0 + i / (rd - rot), j = rot + i % (rd - rot);
        q_wide[((size_t)t * n_heads + h) * wide + rank + j] = row[h * qh + d + j];
    }
    if (blockIdx.y != 0) return;

    // the lists of the grouped products: head h owns the rows h * T .. (h + 1) * T, in tiles of tile_rows
    if (t == 0) {
        for (int h = tid; h <= n_heads; h += blockDim.x) offsets[h] = h * n_tokens;
        const int per_head = (n_tokens + tile_rows - 1) / tile_rows;
        for (int i = tid; i < n_heads * per_head; i += blockDim.x) {
            const int h = i / per_head, k = i % per_head;
            tiles[2 * i] = h;
            tiles[2 * i + 1] = h * n_tokens + k * tile_rows;
        }
        if (tid == 0) n_tiles[0] = n_heads * per_head;
    }
    for (int h = tid; h < n_heads; h += blockDim.x) order[(size_t)h * n_tokens + t] = h * n_tokens + t;
    if (!write_kv) return;

    // the cache row: normalised latent, rotated key part
    const T* lat = row + (size_t)n_heads * qh;
    float ss = 0.f;
    for (int j = tid; j < rank; j += blockDim.x) {
        const float v = to_f32<T>(lat[j]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)rank + eps);
    const int slot = seq_slot[token_seq[t]];
    if (!RI_BLOCK_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT) || !RI_BLOCK_IN_RANGE(pos / page_size, max_pages, RI_CHECK_PAGE_INDEX)) return;
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    if (!RI_BLOCK_IN_LIMIT(page, RI_LIMIT_PAGES, RI_CHECK_PAGE)) return;
    T* dst = cache + ((size_t)page * page_size + (pos % page_size)) * wide;
    for (int j = tid; j < rank; j += blockDim.x) dst[j] = from_f32<T>(to_f32<T>(lat[j]) * scale * c_w[j]);
    for (int k = tid; k < half; k += blockDim.x) {
        const int i0 = style == 0 ? k : 2 * k, i1 = style == 0 ? k + half : 2 * k + 1;
        const float x0 = to_f32<T>(lat[rank + i0]), x1 = to_f32<T>(lat[rank + i1]);
        dst[rank + i0] = from_f32<T>(x0 * c[k] - x1 * s[k]);
        dst[rank + i1] = from_f32<T>(x0 * s[k] + x1 * c[k]);
    }
    for (int j = rot + tid; j < rd; j += blockDim.x) dst[rank + j] = lat[rank + j];
}

template <typename T>
__global__ void latent_widen_kernel(const float* __restrict__ q_lat, T* __restrict__ q_wide, int n_tokens, int n_heads,
                                    int rank, int rd, int vec) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    if (vec) {                      // bf16, rank and rd multiples of 8: eight channels per thread, 16-byte stores
        const int r8 = rank >> 3;
        const size_t total = (size_t)n_tokens * n_heads * r8;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
            const int j = (int)(i % r8) * 8;
            const size_t th = i / r8;
            const int h = (int)(th % n_heads);
            const size_t t = th / n_heads;
            const float4* src = reinterpret_cast<const float4*>(q_lat + ((size_t)h * n_tokens + t) * rank + j);
            const float4 a = src[0], b = src[1];
            __nv_bfloat162 p[4] = {__floats2bfloat162_rn(a.x, a.y), __floats2bfloat162_rn(a.z, a.w),
                                   __floats2bfloat162_rn(b.x, b.y), __floats2bfloat162_rn(b.z, b.w)};
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(q_wide) + th * (rank + rd) + j) = *reinterpret_cast<uint4*>(p);
        }
        return;
    }
    const size_t total = (size_t)n_tokens * n_heads * rank;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int j = (int)(i % rank);
        const size_t th = i / rank;                   // t * heads + h
        const int h = (int)(th % n_heads);
        const size_t t = th / n_heads;
        q_wide[th * (rank + rd) + j] = from_f32<T>(q_lat[((size_t)h * n_tokens + t) * rank + j]);
    }
}

template <typename T>
__global__ void latent_gate_kernel(const float* __restrict__ v, const T* __restrict__ gates, int gate_ld,
                                   T* __restrict__ out, int n_tokens, int n_heads, int vd, int vec) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    if (vec) {                      // bf16, vd a multiple of 8: eight channels per thread, 16-byte stores
        const int v8 = vd >> 3;
        const size_t total = (size_t)n_tokens * n_heads * v8;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
            const int j = (int)(i % v8) * 8;
            const size_t th = i / v8;
            const int h = (int)(th % n_heads);
            const size_t t = th / n_heads;
            float g = 1.f;
            if (gates != nullptr) g = 1.f / (1.f + expf(-to_f32<T>(gates[t * gate_ld + h])));
            const float4* src = reinterpret_cast<const float4*>(v + ((size_t)h * n_tokens + t) * vd + j);
            const float4 a = src[0], b = src[1];
            __nv_bfloat162 p[4] = {__floats2bfloat162_rn(a.x * g, a.y * g), __floats2bfloat162_rn(a.z * g, a.w * g),
                                   __floats2bfloat162_rn(b.x * g, b.y * g), __floats2bfloat162_rn(b.z * g, b.w * g)};
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + th * vd + j) = *reinterpret_cast<uint4*>(p);
        }
        return;
    }
    const size_t total = (size_t)n_tokens * n_heads * vd;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int j = (int)(i % vd);
        const size_t th = i / vd;
        const int h = (int)(th % n_heads);
        const size_t t = th / n_heads;
        float g = 1.f;
        if (gates != nullptr) g = 1.f / (1.f + expf(-to_f32<T>(gates[t * gate_ld + h])));
        out[i] = from_f32<T>(v[((size_t)h * n_tokens + t) * vd + j] * g);
    }
}

int blocks_for(size_t total) {
    const size_t b = (total + 255) / 256;
    return (int)(b < 16384 ? (b ? b : 1) : 16384);
}

}  // namespace

// proj: [T, ld], the heads' queries from column 0, then (write_kv) the latent and its key part.  cache: one layer,
// [pages, 1, page_size, rank + rd].  q_nope [heads, T, d], q_wide [T, heads, rank + rd] (its last rd channels are
// written here).  offsets int32 [heads + 1], order int32 [heads * T], tiles int32 [2 * heads * ceil(T / tile_rows)],
// n_tiles int32 [1].
RI_API int ri_latent_prepare(const void* proj, int dtype, int ld, const float* cos_t, const float* sin_t, const float* c_w,
                             float eps, const int* token_pos, const int* token_seq, const int* seq_slot,
                             const int* page_table, int max_pages, void* cache, void* q_nope, void* q_wide, int* offsets,
                             int* order, int* tiles, int* n_tiles, int n_tokens, int n_heads, int d, int rd, int rank,
                             int rot, int style, int page_size, int write_kv, int tile_rows, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot <= 0) rot = rd;
    if (rot % 2 || rot > rd) return fail("latent_prepare: %d rotated channels of a part of %d", rot, rd);
    if (style != 0 && style != 1) return fail("latent_prepare: unknown style %d", style);
    if (tile_rows <= 0 || n_heads <= 0 || d <= 0 || rank <= 0) return fail("latent_prepare: sizes");
    if ((long long)n_heads * n_tokens > 0x7fffffffLL) return fail("latent_prepare: %d heads x %d tokens exceed 2^31", n_heads, n_tokens);
    const int groups = (n_heads + PREPARE_HEADS - 1) / PREPARE_HEADS;
    if (groups > 65535) return fail("latent_prepare: %d heads exceed the grid limit", n_heads);
    const int vec = dtype == RI_BF16 && d % 8 == 0 && rd % 8 == 0 && ld % 8 == 0 && (uintptr_t)proj % 16 == 0 && (uintptr_t)q_nope % 16 == 0;
    const dim3 grid(n_tokens, groups);
    cudaError_t e;
#define RI_PREPARE(T) launch_dependent(latent_prepare_kernel<T>, grid, dim3(128), (size_t)0, stream, (const T*)proj, ld, cos_t, sin_t, \
        c_w, eps, token_pos, token_seq, seq_slot, page_table, max_pages, (T*)cache, (T*)q_nope, (T*)q_wide, offsets, order, \
        tiles, n_tiles, n_tokens, n_heads, d, rd, rank, rot, style, page_size, write_kv, tile_rows, vec)
    if (dtype == RI_F32) e = RI_PREPARE(float);
    else if (dtype == RI_BF16) e = RI_PREPARE(__nv_bfloat16);
    else return fail("latent_prepare: unknown dtype %d", dtype);
#undef RI_PREPARE
    return check_launch(e, "latent_prepare");
}

RI_API int ri_latent_widen(const float* q_lat, void* q_wide, int dtype, int n_tokens, int n_heads, int rank, int rd,
                           cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int vec = dtype == RI_BF16 && rank % 8 == 0 && rd % 8 == 0 && (uintptr_t)q_lat % 16 == 0 && (uintptr_t)q_wide % 16 == 0;
    const int blocks = blocks_for((size_t)n_tokens * n_heads * rank / (vec ? 8 : 1));
    cudaError_t e;
    if (dtype == RI_F32) e = launch_dependent(latent_widen_kernel<float>, blocks, 256, 0, stream, q_lat, (float*)q_wide, n_tokens, n_heads, rank, rd, 0);
    else if (dtype == RI_BF16) e = launch_dependent(latent_widen_kernel<__nv_bfloat16>, blocks, 256, 0, stream, q_lat, (__nv_bfloat16*)q_wide, n_tokens, n_heads, rank, rd, vec);
    else return fail("latent_widen: unknown dtype %d", dtype);
    return check_launch(e, "latent_widen");
}

RI_API int ri_latent_gate(const float* v, const void* gates, int gate_ld, void* out, int dtype, int n_tokens, int n_heads,
                          int vd, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int vec = dtype == RI_BF16 && vd % 8 == 0 && (uintptr_t)v % 16 == 0 && (uintptr_t)out % 16 == 0;
    const int blocks = blocks_for((size_t)n_tokens * n_heads * vd / (vec ? 8 : 1));
    cudaError_t e;
    if (dtype == RI_F32) e = launch_dependent(latent_gate_kernel<float>, blocks, 256, 0, stream, v, (const float*)gates, gate_ld, (float*)out, n_tokens, n_heads, vd, 0);
    else if (dtype == RI_BF16) e = launch_dependent(latent_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, v, (const __nv_bfloat16*)gates, gate_ld, (__nv_bfloat16*)out, n_tokens, n_heads, vd, vec);
    else return fail("latent_gate: unknown dtype %d", dtype);
    return check_launch(e, "latent_gate");
}

RI_DEFINE_LAST_ERROR()
