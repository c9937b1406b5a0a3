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
//            tokens in order; the state is read first and written last.  Long runs of new tokens are
//            cut into pieces that are scanned side by side (see below), all in float32
//   norm     per (token, head): o / sqrt(mean(o^2) + eps) * w * out_scale -> the run dtype
//
// The projections z = [zq | zf | v] arrive as one float32 matrix [tokens, ld].  What an earlier kernel of the
// step wrote is read after `wait_for_previous_kernels()` through plain pointers (a `const __restrict__` load
// may be moved ahead of the wait).
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

// Threads of a warp: lane = column_in_warp * R + r.  Thread (r, j) keeps ROWS consecutive rows
// (r * ROWS ...) of column j of the state in registers; the sum over rows of S[i, j] q[i] is finished by
// log2(R) shuffles inside the warp.  No block-wide barrier in the loop, and the next token's q, f and v
// are on their way while the current one is worked on.
//
// A long run of new tokens is cut into pieces of `piece` tokens that run side by side (three passes):
//   LOCAL   every piece from a zero state: its end state and the product of its gates go to scratch
//   (carry) per state element, piece after piece: scratch <- the state the piece starts from,
//           running <- gates' product * running + the piece's end state; the slot's state at the end
//   FINAL   every piece again, from its true start state: writes o
// A short run (one piece per sequence: decode steps, small portions) is one pass, WHOLE: from the
// slot's state, writing o and the slot's state.
constexpr int R = 8;                 // row slices per column
constexpr int COLS = 32;             // value columns per block
constexpr int SCAN_THREADS = R * COLS;
enum ScanMode { WHOLE = 0, LOCAL = 1, FINAL = 2 };

template <int ROWS>
struct TokenRegs {
    float f[ROWS], q[ROWS], v;
};

template <int ROWS, bool VEC>
__device__ __forceinline__ void load_token(TokenRegs<ROWS>& reg, const float* row, int q_off, int f_off, int v_off,
                                           int i0, int dim, bool live) {
    if (VEC) {
#pragma unroll
        for (int k = 0; k < ROWS; k += 4) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
            if (i0 + k < dim) {                                   // dim is a multiple of 4 here
                a = *reinterpret_cast<const float4*>(row + f_off + i0 + k);
                b = *reinterpret_cast<const float4*>(row + q_off + i0 + k);
            }
            reg.f[k] = a.x; reg.f[k + 1] = a.y; reg.f[k + 2] = a.z; reg.f[k + 3] = a.w;
            reg.q[k] = b.x; reg.q[k + 1] = b.y; reg.q[k + 2] = b.z; reg.q[k + 3] = b.w;
        }
    } else {
#pragma unroll
        for (int k = 0; k < ROWS; ++k) {
            const bool in = i0 + k < dim;
            reg.f[k] = in ? row[f_off + i0 + k] : 0.f;
            reg.q[k] = in ? row[q_off + i0 + k] : 0.f;
        }
    }
    reg.v = live ? row[v_off] : 0.f;
}

template <int ROWS, bool VEC>
__global__ void __launch_bounds__(SCAN_THREADS, ROWS <= 16 ? 2 : 1)
recurrence_scan_kernel(const float* z, int ld, float* __restrict__ o_raw, float* state,
                       float* piece_state, float* piece_gates, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ seq_slot, int heads, int dim, int vdim, int mode, int piece, int max_pieces) {
    const int b = blockIdx.x / max_pieces, c = blockIdx.x % max_pieces, h = blockIdx.y;
    const int r = threadIdx.x % R;
    const int j = blockIdx.z * COLS + threadIdx.x / R;
    const bool live = j < vdim;
    const int i0 = r * ROWS;
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int t0 = cu_seqlens[b] + c * piece;
    const int seq_end = cu_seqlens[b + 1];
    if (t0 >= seq_end) return;                                   // uniform over the block
    const int t1 = (mode == WHOLE) ? seq_end : min(seq_end, t0 + piece);
    float* S = nullptr;
    if (mode == WHOLE) {
        const int slot = seq_slot[b];
        if (!RI_BLOCK_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT)) return;
        S = state + (((size_t)slot * heads + h) * dim) * vdim;
    } else {
        S = piece_state + (((size_t)blockIdx.x * heads + h) * dim) * vdim;
    }
    float s[ROWS], g[ROWS];
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
        s[k] = (mode != LOCAL && live && i0 + k < dim) ? S[(size_t)(i0 + k) * vdim + j] : 0.f;
        g[k] = 1.f;
    }
    const int qdim = heads * dim;
    const int q_off = h * dim, f_off = qdim + h * dim, v_off = 2 * qdim + h * vdim + j;
    const int o_ld = heads * vdim;
    TokenRegs<ROWS> cur, nxt;
    load_token<ROWS, VEC>(nxt, z + (size_t)t0 * ld, q_off, f_off, v_off, i0, dim, live);
    for (int t = t0; t < t1; ++t) {
        cur = nxt;
        if (t + 1 < t1) load_token<ROWS, VEC>(nxt, z + (size_t)(t + 1) * ld, q_off, f_off, v_off, i0, dim, live);
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int k = 0; k < ROWS; ++k) {
            const float fi = cur.f[k];
            s[k] = fmaf(fi, s[k], fmaf(-fi, cur.v, cur.v));          // f s + (1 - f) v; rows beyond dim: f = 0, q = 0
            if (mode == LOCAL) g[k] *= fi;
            if (k & 1) acc1 = fmaf(s[k], cur.q[k], acc1); else acc0 = fmaf(s[k], cur.q[k], acc0);
        }
        if (mode != LOCAL) {
            float acc = acc0 + acc1;
#pragma unroll
            for (int o = R / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && r == 0) o_raw[(size_t)t * o_ld + h * vdim + j] = acc;
        }
    }
    if (mode != FINAL) {
#pragma unroll
        for (int k = 0; k < ROWS; ++k)
            if (live && i0 + k < dim) S[(size_t)(i0 + k) * vdim + j] = s[k];
    }
    if (mode == LOCAL && blockIdx.z == 0 && threadIdx.x / R == 0) {
        float* G = piece_gates + ((size_t)blockIdx.x * heads + h) * dim;
#pragma unroll
        for (int k = 0; k < ROWS; ++k)
            if (i0 + k < dim) G[i0 + k] = g[k];
    }
}

// Per state element, piece after piece: the state each piece starts from, and the slot's state at the end.
__global__ void recurrence_carry_kernel(float* state, float* piece_state,
                                        const float* piece_gates, const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ seq_slot, int heads, int dim, int vdim, int piece,
                                        int max_pieces) {
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int b = blockIdx.y;
    const size_t per_seq = (size_t)heads * dim * vdim;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per_seq) return;
    const int n_new = cu_seqlens[b + 1] - cu_seqlens[b];
    const int pieces = (n_new + piece - 1) / piece;
    const int slot = seq_slot[b];
    if (!RI_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT)) return;
    const size_t row = e / vdim;                                  // head * dim + channel
    float running = state[(size_t)slot * per_seq + e];
    for (int c = 0; c < pieces; ++c) {
        const size_t at = (size_t)(b * max_pieces + c);
        const float local = piece_state[at * per_seq + e];
        piece_state[at * per_seq + e] = running;
        running = fmaf(piece_gates[at * heads * dim + row], running, local);
    }
    state[(size_t)slot * per_seq + e] = running;
}

// One warp per (token, head): RMS norm over the head's vdim values with one weight shared by heads.
template <typename T>
__global__ void headwise_rmsnorm_kernel(const float* x, int ld, int col0, const float* __restrict__ w,
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


template <int ROWS>
cudaError_t launch_scan(bool vec, dim3 grid, cudaStream_t stream, const float* z, int ld, float* o_raw, float* state,
                        float* piece_state, float* piece_gates, const int* cu_seqlens, const int* seq_slot, int heads, int dim,
                        int vdim, int mode, int piece, int max_pieces) {
    if (vec && ROWS % 4 == 0)
        return launch_dependent(recurrence_scan_kernel<ROWS, (ROWS % 4 == 0)>, grid, SCAN_THREADS, 0, stream, z, ld, o_raw, state,
                                piece_state, piece_gates, cu_seqlens, seq_slot, heads, dim, vdim, mode, piece, max_pieces);
    return launch_dependent(recurrence_scan_kernel<ROWS, false>, grid, SCAN_THREADS, 0, stream, z, ld, o_raw, state,
                            piece_state, piece_gates, cu_seqlens, seq_slot, heads, dim, vdim, mode, piece, max_pieces);
}

}  // namespace

// Floats of scratch a call with pieces needs: [n_seqs * max_pieces] states and gate products.
RI_API long long ri_gated_recurrence_scratch(int n_seqs, int max_pieces, int heads, int dim, int vdim) {
    return (long long)n_seqs * max_pieces * heads * dim * ((long long)vdim + 1);
}

// z: float32 [n_tokens, ld] = [zq (heads*dim) | zf (heads*dim) | v (heads*vdim)]; zq and zf are overwritten
// by q and f.  o_raw: float32 [n_tokens, heads*vdim] scratch.  state: float32 [slots, heads, dim, vdim].
// out: [n_tokens, heads*vdim] in `dtype`.  piece > 0: sequences' new tokens are cut into pieces of that many
// tokens, at most max_pieces per sequence (the longest run of new tokens / piece, rounded up), worked on side
// by side with `scratch` (ri_gated_recurrence_scratch floats); piece == 0: one pass per sequence.
RI_API int ri_gated_recurrence(float* z, int ld, const float* bias, const float* low, const float* norm_w,
                               float* state, const int* cu_seqlens, const int* seq_slot, float* o_raw, void* out, int dtype,
                               int n_tokens, int n_seqs, int heads, int dim, int vdim, float eps, float out_scale,
                               int piece, int max_pieces, float* scratch, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (ld < 2 * heads * dim + heads * vdim) return fail("gated_recurrence: rows of %d values are too short", ld);
    if (heads > 65535) return fail("gated_recurrence: %d heads exceed the grid limit", heads);
    int rows = (dim + R - 1) / R;
    rows = rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : rows <= 32 ? 32 : 64;
    if (dim > 64 * R) return fail("gated_recurrence: a head of %d channels exceeds %d", dim, 64 * R);
    if (piece > 0 && (max_pieces <= 0 || scratch == nullptr)) return fail("gated_recurrence: pieces need scratch");
    const int qdim = heads * dim;
    {
        const size_t total = (size_t)n_tokens * qdim;
        const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
        cudaError_t e = launch_dependent(recurrence_prepare_kernel, blocks, 256, 0, stream, z, ld, bias, low, n_tokens, qdim);
        if (check_launch(e, "gated_recurrence (prepare)")) return 1;
    }
    const bool vec = dim % 4 == 0 && ld % 4 == 0 && (uintptr_t)z % 16 == 0;
    const int col_tiles = (vdim + COLS - 1) / COLS;
    float* piece_state = scratch;
    float* piece_gates = piece > 0 ? scratch + (size_t)n_seqs * max_pieces * heads * dim * vdim : nullptr;
    auto scan = [&](int mode) -> int {
        const int mp = mode == WHOLE ? 1 : max_pieces;
        dim3 grid(n_seqs * mp, heads, col_tiles);
        cudaError_t e;
#define RI_SCAN(ROWS) launch_scan<ROWS>(vec, grid, stream, z, ld, o_raw, state, piece_state, piece_gates, cu_seqlens, seq_slot, \
                                        heads, dim, vdim, mode, piece > 0 ? piece : 1, mp)
        if (rows == 4) e = RI_SCAN(4);
        else if (rows == 8) e = RI_SCAN(8);
        else if (rows == 16) e = RI_SCAN(16);
        else if (rows == 32) e = RI_SCAN(32);
        else e = RI_SCAN(64);
#undef RI_SCAN
        return check_launch(e, "gated_recurrence (scan)");
    };
    if (piece <= 0) {
        if (scan(WHOLE)) return 1;
    } else {
        if (scan(LOCAL)) return 1;
        const size_t per_seq = (size_t)heads * dim * vdim;
        dim3 grid((unsigned)((per_seq + 255) / 256), n_seqs);
        cudaError_t e = launch_dependent(recurrence_carry_kernel, grid, 256, 0, stream, state, piece_state,
                                         (const float*)piece_gates, cu_seqlens, seq_slot, heads, dim, vdim, piece, max_pieces);
        if (check_launch(e, "gated_recurrence (carry)")) return 1;
        if (scan(FINAL)) return 1;
    }
    {
        const long long warps = (long long)n_tokens * heads;
        const int blocks = (int)((warps * 32 + 255) / 256);
        cudaError_t e;
        if (dtype == RI_F32)
            e = launch_dependent(headwise_rmsnorm_kernel<float>, blocks, 256, 0, stream, (const float*)o_raw, heads * vdim, 0, norm_w,
                                 (float*)out, heads * vdim, n_tokens, heads, vdim, eps, out_scale);
        else if (dtype == RI_BF16)
            e = launch_dependent(headwise_rmsnorm_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const float*)o_raw, heads * vdim, 0,
                                 norm_w, (__nv_bfloat16*)out, heads * vdim, n_tokens, heads, vdim, eps, out_scale);
        else
            return fail("gated_recurrence: unknown dtype %d", dtype);
        return check_launch(e, "gated_recurrence (norm)");
    }
}

RI_DEFINE_LAST_ERROR()
