// Attention of many query heads over ONE cached row per position (attention over a shared latent), bf16, on the
// tensor cores (mma.sync m16n8k16, float32 accumulation, float32 softmax).
//
// A position's cached row holds KD = RANK + RD channels; it is the key of every head, and its first RANK
// channels are the value of every head.  The queries come as rows of KD channels, one per (token, head), token
// by token: row t * heads + h.  Because all heads read the same keys, the heads of a token (and of its
// neighbours) are simply more query ROWS of one problem: a CTA takes BM = 128 consecutive rows of one sequence
// (64 when the step's sequences bring fewer), a warp 16 of them, and walks the sequence's keys 32 at a time
// (half a cache page), causal per row.  Shapes per warp
// and key tile: S[16 x 32] = Q[16 x KD] K^T (KD / 16 k-steps), then O[16 x NV] += P[16 x 32] V[32 x NV].
//
// NV is what a thread can hold of O in registers: 256 value channels (128 registers).  A latent of 512 channels
// is therefore cut into two halves that run as two CTAs (blockIdx.z); each recomputes the scores (1.5 x the
// multiply-adds of one pass, and no exchange between CTAs).
//
// Steps of few rows (decoding) cut the keys into `n_splits` runs as well: every run writes an un-normalised
// partial result with its (max, sum) to scratch, and a second kernel merges them by log-sum-exp.
//
// Q and the key tiles sit in shared memory with rows padded by 16 bytes (conflict-free ldmatrix); key tiles are
// double-buffered with cp.async.  The result is written head-major, [heads, tokens, RANK]: the rows of the
// per-head up-projection that follows.
#include "common.cuh"

using namespace ri;

namespace {

constexpr int PAGE = 64;
constexpr int BN = 32;              // keys per tile

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void st_zero16(uint32_t dst) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int RANK, int RD, int NZ, int BM>
__global__ void __launch_bounds__(BM * 2, 1)
latent_attn_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                   const int* __restrict__ page_table, int max_pages, const int* __restrict__ seq_slot,
                   const int* __restrict__ seq_start, const int* __restrict__ cu_seqlens, int n_heads, int n_tokens,
                   float scale_log2, int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                   __nv_bfloat16* __restrict__ out) {
    constexpr int KD = RANK + RD;
    constexpr int ROW = (KD + 8) * 2;                 // bytes of a padded row in shared memory
    constexpr int NV = RANK / NZ;                     // value channels of this CTA
    constexpr int KSTEPS = KD / 16, NT_O = NV / 8;
    constexpr int THREADS = BM * 2;                   // a warp per 16 rows
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t q_s = smem_u32(smem);              // [BM][KD + 8]
    const uint32_t k_s = q_s + BM * ROW;              // 2 x [BN][KD + 8]

    const int b = blockIdx.y / n_splits, split = blockIdx.y % n_splits;
    const int z0 = blockIdx.z * NV;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    let_next_kernel_start();
    wait_for_previous_kernels();                      // the queries and the step's new cache rows come from the kernels before
    const int tok0 = cu_seqlens[b], n_rows = (cu_seqlens[b + 1] - tok0) * n_heads;
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;          // the longest tiles first
    const int r0 = tile * BM;
    if (r0 >= n_rows) return;
    const int start = seq_start[b];
    const int last_row = min(n_rows, r0 + BM) - 1;
    const int n_keys = start + last_row / n_heads + 1;              // the keys the tile's last row sees
    const int n_kt = (n_keys + BN - 1) / BN;
    const int per = (n_kt + n_splits - 1) / n_splits;
    const int kt_begin = split * per, kt_end = min(n_kt, kt_begin + per);
    const int* pages = page_table + (size_t)seq_slot[b] * max_pages;
    const size_t row_base = (size_t)tok0 * n_heads + r0;            // first query row of the tile

    auto load_keys = [&](int kt, int stage) {
        const int j0 = kt * BN;
        const int page = pages[j0 / PAGE];
        const __nv_bfloat16* src = cache + ((size_t)page * PAGE + (j0 % PAGE)) * KD;
        const uint32_t dst = k_s + stage * (BN * ROW);
        for (int i = tid; i < BN * (KD / 8); i += THREADS) {
            const int r = i / (KD / 8), c = i % (KD / 8);
            if (j0 + r < n_keys) cp_async16(dst + r * ROW + c * 16, src + (size_t)r * KD + c * 8);
            else st_zero16(dst + r * ROW + c * 16);
        }
    };

    // the queries of the tile (rows beyond the sequence's: zeros), and the first key tile
    for (int i = tid; i < BM * (KD / 8); i += THREADS) {
        const int r = i / (KD / 8), c = i % (KD / 8);
        if (r0 + r < n_rows) cp_async16(q_s + r * ROW + c * 16, q + (row_base + r) * KD + c * 8);
        else st_zero16(q_s + r * ROW + c * 16);
    }
    if (kt_begin < kt_end) load_keys(kt_begin, 0);
    cp_async_commit();

    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    // the positions of this thread's two rows
    const int row_lo = r0 + warp * 16 + (lane >> 2), row_hi = row_lo + 8;
    const int pos_lo = start + row_lo / n_heads, pos_hi = start + row_hi / n_heads;

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int stage = (kt - kt_begin) & 1;
        if (kt + 1 < kt_end) load_keys(kt + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t kb = k_s + stage * (BN * ROW);
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll 4
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(q_s + (warp * 16 + (lane & 15)) * ROW + (ks * 16 + (lane >> 4) * 8) * 2, a0, a1, a2, a3);
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(kb + (np * 16 + (lane & 7) + (lane >> 4) * 8) * ROW + (ks * 16 + ((lane >> 3) & 1) * 8) * 2, b0, b1, b2, b3);
                mma_bf16(s[2 * np], a0, a1, a2, a3, b0, b1);
                mma_bf16(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // causal mask per row, in units of log2
        const int j0 = kt * BN + (lane & 3) * 2;
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = j0 + nt * 8 + e;
                s[nt][e] = j <= pos_lo ? s[nt][e] * scale_log2 : -INFINITY;
                s[nt][2 + e] = j <= pos_hi ? s[nt][2 + e] * scale_log2 : -INFINITY;
                mx_lo = fmaxf(mx_lo, s[nt][e]);
                mx_hi = fmaxf(mx_hi, s[nt][2 + e]);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo, base_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float al_lo = exp2f(m_lo - base_lo), al_hi = exp2f(m_hi - base_hi);     // exp2(-inf) = 0 at the first tile
        m_lo = mn_lo;
        m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s[nt][e] = exp2f(s[nt][e] - base_lo);
                s[nt][2 + e] = exp2f(s[nt][2 + e] - base_hi);
                sum_lo += s[nt][e];
                sum_hi += s[nt][2 + e];
            }
        }
        l_lo = l_lo * al_lo + sum_lo;
        l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
            o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi;
        }
        // O += P V: the values are the first channels of the key rows
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            const uint32_t a0 = pack2(s[2 * kk][0], s[2 * kk][1]), a1 = pack2(s[2 * kk][2], s[2 * kk][3]);
            const uint32_t a2 = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < NT_O / 2; ++dp) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(kb + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ROW + (z0 + dp * 16 + (lane >> 4) * 8) * 2,
                                  b0, b1, b2, b3);
                mma_bf16(o[2 * dp], a0, a1, a2, a3, b0, b1);
                mma_bf16(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();              // the stage is free for the tile after next
    }
    cp_async_wait<0>();

    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const int col = z0 + (lane & 3) * 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = half ? row_hi : row_lo;
        if (r >= n_rows) continue;
        const size_t g = (size_t)tok0 * n_heads + r;                 // global query row: token * heads + head
        const float l = half ? l_hi : l_lo, m = half ? m_hi : m_lo;
        if (n_splits == 1) {
            const float inv = 1.f / l;
            const size_t t = g / n_heads, h = g % n_heads;
            __nv_bfloat16* dst = out + (h * (size_t)n_tokens + t) * RANK + col;
#pragma unroll
            for (int i = 0; i < NT_O; ++i)
                *reinterpret_cast<uint32_t*>(dst + i * 8) = pack2(o[i][2 * half] * inv, o[i][2 * half + 1] * inv);
        } else {
            float* dst = part_o + (g * n_splits + split) * RANK + col;
#pragma unroll
            for (int i = 0; i < NT_O; ++i)
                *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2 * half], o[i][2 * half + 1]);
            if (blockIdx.z == 0 && (lane & 3) == 0) {
                part_ml[(g * n_splits + split) * 2] = m;
                part_ml[(g * n_splits + split) * 2 + 1] = l;
            }
        }
    }
}

// out[h, t, :] = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s over the runs of keys; a block per query row
__global__ void latent_attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int n_heads,
                                           int n_tokens, int rank, int n_splits, __nv_bfloat16* __restrict__ out) {
    const size_t g = blockIdx.x;
    let_next_kernel_start();
    wait_for_previous_kernels();
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(g * n_splits + s) * 2]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_ml[(g * n_splits + s) * 2];
        if (ms != -INFINITY) L += exp2f(ms - M) * part_ml[(g * n_splits + s) * 2 + 1];
    }
    const float inv = 1.f / L;
    const size_t t = g / n_heads, h = g % n_heads;
    __nv_bfloat16* dst = out + (h * (size_t)n_tokens + t) * rank;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[(g * n_splits + s) * 2];
            if (ms != -INFINITY) acc += exp2f(ms - M) * part_o[(g * n_splits + s) * rank + d];
        }
        dst[d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int RANK, int RD, int BM>
int launch(const void* q, const void* cache, const int* page_table, int max_pages, const int* seq_slot, const int* seq_start,
           const int* cu_seqlens, int n_seqs, int max_new, int n_heads, int n_tokens, float scale, int n_splits, float* part_o,
           float* part_ml, void* out, cudaStream_t stream) {
    constexpr int NZ = RANK > 256 ? 2 : 1;
    constexpr int KD = RANK + RD;
    constexpr int SMEM = (BM + 2 * BN) * (KD + 8) * 2;
    static_assert(SMEM <= 227 * 1024, "the tile does not fit shared memory");
    auto kernel = latent_attn_kernel<RANK, RD, NZ, BM>;
    static PerDeviceOnce configured;
    if (int rc = raise_dynamic_smem(kernel, SMEM, configured, "latent attention")) return rc;
    const int tiles = (int)(((long long)max_new * n_heads + BM - 1) / BM);
    dim3 grid(tiles, n_seqs * n_splits, NZ);
    cudaError_t e = launch_dependent(kernel, grid, dim3(BM * 2), (size_t)SMEM, stream, (const __nv_bfloat16*)q,
                                     (const __nv_bfloat16*)cache, page_table, max_pages, seq_slot, seq_start, cu_seqlens, n_heads,
                                     n_tokens, scale * 1.4426950408889634f, n_splits, part_o, part_ml, (__nv_bfloat16*)out);
    if (int rc = check_launch(e, "latent_attention")) return rc;
    if (n_splits > 1) {
        e = launch_dependent(latent_attn_combine_kernel, dim3((unsigned)((long long)n_tokens * n_heads)), dim3(RANK >= 256 ? 128 : 64),
                             (size_t)0, stream, (const float*)part_o, (const float*)part_ml, n_heads, n_tokens, (int)RANK, n_splits,
                             (__nv_bfloat16*)out);
        return check_launch(e, "latent_attention_combine");
    }
    return 0;
}

}  // namespace

// rows of queries a CTA takes in a step whose longest run of new rows is `rows` (the host plans its runs of keys with it)
RI_API int ri_latent_attention_mma_tile_rows(long long rows) { return rows >= 128 ? 128 : 64; }

// 1 if the kernel is built for these sizes (bf16 only; pages of 64 positions)
RI_API int ri_latent_attention_mma_supports(int rank, int rd, int page_size) {
    return page_size == PAGE && (rank == 64 || rank == 128 || rank == 256 || rank == 512) && (rd == 32 || rd == 64);
}

// q: bf16 [n_tokens * n_heads, rank + rd], rows token by token, a token's heads together.  cache: one layer,
// bf16 [pages, 1, 64, rank + rd].  out: bf16 [n_heads, n_tokens, rank].  n_splits > 1: part_o float32
// [n_tokens * n_heads * n_splits * rank], part_ml float32 [n_tokens * n_heads * n_splits * 2].
RI_API int ri_latent_attention_mma(const void* q, const void* cache, const int* page_table, int max_pages, const int* seq_slot,
                                   const int* seq_start, const int* cu_seqlens, int n_seqs, int max_new, int n_heads,
                                   int n_tokens, int rank, int rd, float scale, int n_splits, float* part_o, float* part_ml,
                                   void* out, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (n_splits < 1 || (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)))
        return fail("latent_attention: %d runs of keys need scratch for their partial results", n_splits);
    if ((long long)n_seqs * n_splits > 65535) return fail("latent_attention: %d sequences x %d runs exceed the grid limit", n_seqs, n_splits);
    const bool big = ri_latent_attention_mma_tile_rows((long long)max_new * n_heads) == 128;
#define RI_LATENT(R, D) if (rank == R && rd == D) return big \
        ? launch<R, D, 128>(q, cache, page_table, max_pages, seq_slot, seq_start, cu_seqlens, n_seqs, max_new, n_heads, n_tokens, scale, \
                            n_splits, part_o, part_ml, out, stream) \
        : launch<R, D, 64>(q, cache, page_table, max_pages, seq_slot, seq_start, cu_seqlens, n_seqs, max_new, n_heads, n_tokens, scale, \
                           n_splits, part_o, part_ml, out, stream)
    RI_LATENT(64, 32); RI_LATENT(64, 64); RI_LATENT(128, 32); RI_LATENT(128, 64);
    RI_LATENT(256, 32); RI_LATENT(256, 64); RI_LATENT(512, 32); RI_LATENT(512, 64);
#undef RI_LATENT
    return fail("latent_attention: no tensor-core kernel for a latent of %d + %d channels", rank, rd);
}

RI_DEFINE_LAST_ERROR()
