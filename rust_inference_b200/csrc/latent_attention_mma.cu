// Attention of many query heads over ONE cached row per position (attention over a shared latent), bf16, on the
// tensor cores (mma.sync m16n8k16, float32 accumulation, float32 softmax).
//
// A position's cached row holds KD = RANK + RD channels; it is the key of every head, and its first RANK
// channels are the value of every head.  The queries come as rows of KD channels, one per (token, head), token
// by token: row t * heads + h.  Because all heads read the same keys, the heads of a token (and of its
// neighbours) are simply more query ROWS of one problem: a CTA takes BM consecutive rows of one sequence (128 in
// long steps of narrow latents, else 64; 32 or 16 when no sequence brings more rows, as in decoding, where small
// CTAs in many runs of keys fill the GPU), a warp 16 of them, and walks the sequence's keys 32 at a time
// (half a cache page), causal per row.  Shapes per warp
// and key tile: S[16 x 32] = Q[16 x KD] K^T (KD / 16 k-steps), then O[16 x NV] += P[16 x 32] V[32 x NV].
//
// NV is what a thread can hold of O in registers: 256 value channels (128 registers).  A latent of 512 channels
// is therefore shared by PAIRS of warps: both warps of a pair own the same 16 rows; each computes the scores of
// half of the tile's keys (16 of 32), they exchange row maxima and their halves of P through shared memory (two
// named barriers of 64 threads per tile), and each multiplies the whole P by its half of the value channels.  No
// score is computed twice; a CTA of 64 rows has 8 warps.
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

__device__ __forceinline__ void pair_barrier(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

// NZ = 1: a warp per 16 rows owns all value channels.  NZ = 2: two warps per 16 rows (see above).
template <int RANK, int RD, int NZ, int BM>
__global__ void __launch_bounds__(BM * 2 * NZ, 1)
latent_attn_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                   const int* __restrict__ page_table, int max_pages, const int* __restrict__ seq_slot,
                   const int* __restrict__ seq_start, const int* __restrict__ cu_seqlens, int n_heads, int n_tokens,
                   float scale_log2, int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                   __nv_bfloat16* __restrict__ out) {
    constexpr int KD = RANK + RD;
    constexpr int ROW = (KD + 8) * 2;                 // bytes of a padded row in shared memory
    constexpr int NV = RANK / NZ;                     // value channels of this CTA
    constexpr int KSTEPS = KD / 16, NT_O = NV / 8;
    constexpr int THREADS = BM * 2 * NZ;              // a warp, or a pair of warps, per 16 rows
    constexpr bool PAIR = NZ == 2;
    constexpr int GROUPS = BM / 16;                   // groups of 16 rows
    constexpr int NT_S = PAIR ? 2 : 4;                // tiles of 8 keys whose scores a warp computes
    __shared__ float pair_max[2][PAIR ? GROUPS : 1][16];      // row maxima (and, at the end, row sums) of each half
    __shared__ uint4 pair_p[2][PAIR ? GROUPS : 1][32];        // each half's P as the lanes' A fragments
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t q_s = smem_u32(smem);              // [BM][KD + 8]
    const uint32_t k_s = q_s + BM * ROW;              // 2 x [BN][KD + 8]

    const int b = blockIdx.y / n_splits, split = blockIdx.y % n_splits;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rw = PAIR ? warp % GROUPS : warp;       // which 16 rows
    const int half = PAIR ? warp / GROUPS : 0;        // which half of the keys' scores and of the value channels
    const int z0 = half * NV;
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
        int page = pages[j0 / PAGE];
        if (!RI_IN_LIMIT(page, RI_LIMIT_PAGES, RI_CHECK_PAGE)) page = 0;      // checked build: recorded, read from a page that exists
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
    const int row_lo = r0 + rw * 16 + (lane >> 2), row_hi = row_lo + 8;
    const int pos_lo = start + row_lo / n_heads, pos_hi = start + row_hi / n_heads;

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int stage = (kt - kt_begin) & 1;
        if (kt + 1 < kt_end) load_keys(kt + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t kb = k_s + stage * (BN * ROW);
        float s[NT_S][4];
#pragma unroll
        for (int i = 0; i < NT_S; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        const int key0 = PAIR ? half * 16 : 0;        // the first key of the tile whose score this warp computes
        // a pair's warp has only two tiles of 8 keys, that is two chains of dependent MMAs: the odd k-steps get
        // accumulators of their own (four chains), added below
        float sx[PAIR ? NT_S : 1][4];
        if (PAIR) {
#pragma unroll
            for (int i = 0; i < NT_S; ++i) sx[i][0] = sx[i][1] = sx[i][2] = sx[i][3] = 0.f;
        }
        auto k_step = [&](int ks, float (*acc)[4]) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(q_s + (rw * 16 + (lane & 15)) * ROW + (ks * 16 + (lane >> 4) * 8) * 2, a0, a1, a2, a3);
#pragma unroll
            for (int np = 0; np < NT_S / 2; ++np) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(kb + (key0 + np * 16 + (lane & 7) + (lane >> 4) * 8) * ROW + (ks * 16 + ((lane >> 3) & 1) * 8) * 2, b0, b1, b2, b3);
                mma_bf16(acc[2 * np], a0, a1, a2, a3, b0, b1);
                mma_bf16(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
            }
        };
        static_assert(KSTEPS % 2 == 0, "key rows are a multiple of 32 channels");
#pragma unroll 2
        for (int ks = 0; ks < KSTEPS; ks += 2) {
            k_step(ks, s);
            k_step(ks + 1, PAIR ? sx : s);
        }
        if (PAIR) {
#pragma unroll
            for (int i = 0; i < NT_S; ++i) {
                s[i][0] += sx[i][0]; s[i][1] += sx[i][1]; s[i][2] += sx[i][2]; s[i][3] += sx[i][3];
            }
        }
        // causal mask per row, in units of log2
        const int j0 = kt * BN + key0 + (lane & 3) * 2;
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < NT_S; ++nt) {
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
        if (PAIR) {                   // the maxima over the other half of the keys come from the partner
            if ((lane & 3) == 0) {
                pair_max[half][rw][lane >> 2] = mx_lo;
                pair_max[half][rw][(lane >> 2) + 8] = mx_hi;
            }
            pair_barrier(1 + rw);
            mx_lo = fmaxf(mx_lo, pair_max[half ^ 1][rw][lane >> 2]);
            mx_hi = fmaxf(mx_hi, pair_max[half ^ 1][rw][(lane >> 2) + 8]);
        }
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo, base_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float al_lo = exp2f(m_lo - base_lo), al_hi = exp2f(m_hi - base_hi);     // exp2(-inf) = 0 at the first tile
        m_lo = mn_lo;
        m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT_S; ++nt) {
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
        uint4 p_other = make_uint4(0u, 0u, 0u, 0u);
        if (PAIR) {                   // this warp's 16 keys of P to the partner, the partner's to this warp
            pair_p[half][rw][lane] = make_uint4(pack2(s[0][0], s[0][1]), pack2(s[0][2], s[0][3]), pack2(s[1][0], s[1][1]),
                                                pack2(s[1][2], s[1][3]));
            pair_barrier(1 + rw);
            p_other = pair_p[half ^ 1][rw][lane];
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            uint32_t a0, a1, a2, a3;
            if (PAIR && kk != half) {
                a0 = p_other.x; a1 = p_other.y; a2 = p_other.z; a3 = p_other.w;
            } else {
                const int n0 = PAIR ? 0 : 2 * kk;
                a0 = pack2(s[n0][0], s[n0][1]); a1 = pack2(s[n0][2], s[n0][3]);
                a2 = pack2(s[n0 + 1][0], s[n0 + 1][1]); a3 = pack2(s[n0 + 1][2], s[n0 + 1][3]);
            }
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
    if (PAIR) {                       // a row's sum is the two halves' (their maxima agree tile by tile)
        if ((lane & 3) == 0) {
            pair_max[half][rw][lane >> 2] = l_lo;
            pair_max[half][rw][(lane >> 2) + 8] = l_hi;
        }
        pair_barrier(1 + rw);
        l_lo += pair_max[half ^ 1][rw][lane >> 2];
        l_hi += pair_max[half ^ 1][rw][(lane >> 2) + 8];
    }
    const int col = z0 + (lane & 3) * 2;
#pragma unroll
    for (int hi = 0; hi < 2; ++hi) {
        const int r = hi ? row_hi : row_lo;
        if (r >= n_rows) continue;
        const size_t g = (size_t)tok0 * n_heads + r;                 // global query row: token * heads + head
        const float l = hi ? l_hi : l_lo, m = hi ? m_hi : m_lo;
        if (n_splits == 1) {
            const float inv = 1.f / l;
            const size_t t = g / n_heads, h = g % n_heads;
            __nv_bfloat16* dst = out + (h * (size_t)n_tokens + t) * RANK + col;
#pragma unroll
            for (int i = 0; i < NT_O; ++i)
                *reinterpret_cast<uint32_t*>(dst + i * 8) = pack2(o[i][2 * hi] * inv, o[i][2 * hi + 1] * inv);
        } else {
            float* dst = part_o + (g * n_splits + split) * RANK + col;
#pragma unroll
            for (int i = 0; i < NT_O; ++i)
                *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2 * hi], o[i][2 * hi + 1]);
            if (half == 0 && (lane & 3) == 0) {
                part_ml[(g * n_splits + split) * 2] = m;
                part_ml[(g * n_splits + split) * 2 + 1] = l;
            }
        }
    }
}

// out[h, t, :] = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s over the runs of keys; a block per query row.  The
// runs' (max, sum) pairs are read by the first warp side by side (a loop that folded them one by one would wait
// for one load after the other), their weights go through shared memory, and a thread sums four channels.
constexpr int MAX_RUNS = 32;
__global__ void latent_attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int n_heads,
                                           int n_tokens, int rank, int n_splits, __nv_bfloat16* __restrict__ out) {
    __shared__ float weight[MAX_RUNS];
    const size_t g = blockIdx.x;
    let_next_kernel_start();
    wait_for_previous_kernels();
    if (threadIdx.x < 32) {
        const int s = threadIdx.x;
        float m = -INFINITY, l = 0.f;
        if (s < n_splits) {
            const float2 ml = *reinterpret_cast<const float2*>(part_ml + (g * n_splits + s) * 2);
            m = ml.x;
            l = ml.y;
        }
        const float M = warp_max(m);
        const float w = m == -INFINITY ? 0.f : exp2f(m - M);
        const float L = warp_sum(w * l);
        if (s < n_splits) weight[s] = w / L;
    }
    __syncthreads();
    const size_t t = g / n_heads, h = g % n_heads;
    __nv_bfloat16* dst = out + (h * (size_t)n_tokens + t) * rank;
    const float* src = part_o + g * n_splits * rank;
    for (int d = threadIdx.x * 4; d < rank; d += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int s = 0; s < n_splits; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(src + (size_t)s * rank + d);
            const float w = weight[s];
            acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
        }
        uint2 packed;
        packed.x = pack2(acc.x, acc.y);
        packed.y = pack2(acc.z, acc.w);
        *reinterpret_cast<uint2*>(dst + d) = packed;
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
    dim3 grid(tiles, n_seqs * n_splits, 1);
    cudaError_t e = launch_dependent(kernel, grid, dim3(BM * 2 * NZ), (size_t)SMEM, stream, (const __nv_bfloat16*)q,
                                     (const __nv_bfloat16*)cache, page_table, max_pages, seq_slot, seq_start, cu_seqlens, n_heads,
                                     n_tokens, scale * 1.4426950408889634f, n_splits, part_o, part_ml, (__nv_bfloat16*)out);
    if (int rc = check_launch(e, "latent_attention")) return rc;
    if (n_splits > 1) {
        e = launch_dependent(latent_attn_combine_kernel, dim3((unsigned)((long long)n_tokens * n_heads)), dim3(RANK >= 512 ? 128 : (RANK >= 256 ? 64 : 32)),
                             (size_t)0, stream, (const float*)part_o, (const float*)part_ml, n_heads, n_tokens, (int)RANK, n_splits,
                             (__nv_bfloat16*)out);
        return check_launch(e, "latent_attention_combine");
    }
    return 0;
}

__host__ int tile_rows_for(long long rows, int rank) {
    if (rows <= 16) return 16;
    if (rows <= 32) return 32;
    return rank <= 256 && rows >= 128 ? 128 : 64;
}

template <int RANK, int RD>
int pick(int bm, const void* q, const void* cache, const int* page_table, int max_pages, const int* seq_slot, const int* seq_start,
         const int* cu_seqlens, int n_seqs, int max_new, int n_heads, int n_tokens, float scale, int n_splits, float* part_o,
         float* part_ml, void* out, cudaStream_t stream) {
#define RI_TILE(BM) launch<RANK, RD, BM>(q, cache, page_table, max_pages, seq_slot, seq_start, cu_seqlens, n_seqs, max_new, n_heads, \
                                         n_tokens, scale, n_splits, part_o, part_ml, out, stream)
    if constexpr (RANK <= 256) {
        if (bm == 128) return RI_TILE(128);
    }
    if (bm == 16) return RI_TILE(16);
    if (bm == 32) return RI_TILE(32);
    return RI_TILE(64);
#undef RI_TILE
}

}  // namespace

// rows of queries a CTA takes in a step whose longest run of new rows is `rows` (the host plans its runs of keys with it)
// (a latent of more than 256 channels: at most 64, two warps per 16 rows)
RI_API int ri_latent_attention_mma_tile_rows(long long rows, int rank) { return tile_rows_for(rows, rank); }

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
    if (n_splits > MAX_RUNS) return fail("latent_attention: %d runs of keys exceed %d", n_splits, MAX_RUNS);
    if (n_splits < 1 || (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)))
        return fail("latent_attention: %d runs of keys need scratch for their partial results", n_splits);
    if ((long long)n_seqs * n_splits > 65535) return fail("latent_attention: %d sequences x %d runs exceed the grid limit", n_seqs, n_splits);
    const int bm = tile_rows_for((long long)max_new * n_heads, rank);
#define RI_LATENT(R, D) if (rank == R && rd == D) return pick<R, D>(bm, q, cache, page_table, max_pages, seq_slot, seq_start, cu_seqlens, \
        n_seqs, max_new, n_heads, n_tokens, scale, n_splits, part_o, part_ml, out, stream)
    RI_LATENT(64, 32); RI_LATENT(64, 64); RI_LATENT(128, 32); RI_LATENT(128, 64);
    RI_LATENT(256, 32); RI_LATENT(256, 64); RI_LATENT(512, 32); RI_LATENT(512, 64);
#undef RI_LATENT
    return fail("latent_attention: no tensor-core kernel for a latent of %d + %d channels", rank, rd);
}

RI_DEFINE_LAST_ERROR()
