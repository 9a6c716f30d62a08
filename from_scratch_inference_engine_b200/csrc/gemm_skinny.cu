// Matrix product for steps of few tokens against a small matrix:
// y[T, N] = x[T, K] * w[N, K]^T (+ bias), T <= 16, bfloat16 operands, 32-bit accumulation.
//
// For the q,k,v and o projections of a decode step (25-33 MB of weights) the product is over
// before a pipeline of TMA stages and tensor-memory accumulators has filled: what counts is how
// soon the first bytes are asked for and how many are in flight.  So this kernel has no set-up:
// a block owns 16 rows of w, its 8 warps take turns along k in chunks of 32 elements, every
// lane asks for its 16 bytes of two rows with cp.async into a slot of its own (eight chunks
// ahead, no registers tied up, three blocks per SM: ~190 KB in flight per SM), and
// the tokens are the N side of mma.sync m16n8k16 (8 tokens per instruction).  The order of the
// k elements inside a chunk does not matter to a dot product, so a lane's 16 contiguous bytes
// serve as its fragments of two MMAs as they are, and x gives the matching 16 bytes (read from
// global memory too: the few KB of x stay in L1 / L2).  The eight warps' partial sums meet in
// shared memory.
//
// Launched as a programmatic dependent: the first weights are asked for before the kernel that
// produces x has finished.
#include "common.cuh"

namespace fsie {

constexpr int SK_ROWS = 16;          // rows of w per block (MMA M)
constexpr int SK_WARPS = 16;
constexpr int SK_CHUNK = 32;         // k elements per warp and step: 4 lanes x 16 bytes per row
constexpr int SK_AHEAD = 4;          // chunks whose weights a warp has asked for (a ring of 4 KB per warp)

struct SkinnyParams {
    const bf16* w; const bf16* x; long long ldx;
    void* y; long long ldy; const bf16* bias;
    int T, N, K, out_f32;
};

// The q, k, v product of an attention layer with what follows it on the way to the cache: w
// holds `heads` query heads, then `kv_heads` key heads, then as many value heads, of head_dim
// rows each.  Query and key heads are rotated by the angles of their token's position
// (pairs (i, i + head_dim / 2), cos | sin table as in rope_kv_write), queries go to y, keys
// and values into their token's slot of the pages (slot_of < 0 or no pages: not stored).
struct SkinnyRope {
    const int* positions; const float* cos_sin; int table_len;
    const int* slot_of; bf16* k_pages; bf16* v_pages; long long page_stride; int page_size;
    int heads, kv_heads, head_dim;
    int* error;
};

__device__ __forceinline__ void mma_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// TT: token tiles of 8 (1 or 2).  Dynamic shared memory: per warp a ring of SK_AHEAD slots of 1 KB
// (each lane's 16 bytes of its two rows: a lane reads back only what it asked for itself, so
// no barrier guards the ring); static: the warps' partial sums.
// ROPE: the block's 16 rows are 8 rows of a head and the 8 rows half a head further on - the
// two halves of 8 rotation pairs - and the epilogue is the one SkinnyRope describes.
template <int TT, bool ROPE>
__global__ void __launch_bounds__(32 * SK_WARPS, 2)       // two blocks per SM: 64 registers at most
gemm_skinny_kernel(const SkinnyParams p, const SkinnyRope rope) {
    extern __shared__ __align__(16) unsigned char sk_ring[];
    __shared__ float red[SK_WARPS * SK_ROWS * 8 * TT];            // [warp][16 rows][8 * TT]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int chunks = p.K / SK_CHUNK;
    // rows of w behind rows 0-7 and 8-15 of the block's tile
    int row0, row8;
    if (ROPE) {
        const int per_head = rope.head_dim / 16;                  // blocks per head
        const int head = blockIdx.x / per_head, d0 = (blockIdx.x - head * per_head) * 8;
        row0 = head * rope.head_dim + d0;
        row8 = row0 + rope.head_dim / 2;
    } else {
        row0 = blockIdx.x * SK_ROWS;
        row8 = row0 + 8;
    }
    // this lane's two rows (clamped at the matrix's end; those results are not stored)
    const bf16* w_lo = p.w + (size_t)min(row0 + g, p.N - 1) * p.K + 8 * t;
    const bf16* w_hi = p.w + (size_t)min(row8 + g, p.N - 1) * p.K + 8 * t;
    unsigned char* mine = sk_ring + (size_t)warp * SK_AHEAD * 1024 + lane * 16;     // slot s: + s * 1024; second row: + 512

    auto ask = [&](int slot, int c) {                             // this lane's 32 bytes of chunk c
        if (c < chunks) {
            cp_async_16(mine + slot * 1024, w_lo + c * SK_CHUNK);
            cp_async_16(mine + slot * 1024 + 512, w_hi + c * SK_CHUNK);
        }
        cp_async_commit();                                        // one group per slot, also when empty
    };
#pragma unroll
    for (int j = 0; j < SK_AHEAD; ++j) ask(j, warp + j * SK_WARPS);    // weights do not depend on the kernel before
    // Nor does what the epilogue's rotation needs: the token's position and slot were staged before
    // the step, the table and the bias are constants.  A thread of the epilogue owns one rotation
    // pair of one token (the block has more threads than such pairs) and fetches its angle now.
    constexpr int TP = 8 * TT;
    static_assert(8 * TP <= 32 * SK_WARPS, "one rotation pair per thread");
    int early_pos = 0, early_slot = -1;
    float early_cos = 1.f, early_sin = 0.f, early_bias_lo = 0.f, early_bias_hi = 0.f;
    if (ROPE) {
        const int token = threadIdx.x >> 3, r = threadIdx.x & 7;
        if (threadIdx.x < 8 * TP && token < p.T) {
            const int per_head = rope.head_dim / 16;
            const int head = blockIdx.x / per_head, d = (blockIdx.x - head * per_head) * 8 + r;
            early_pos = rope.positions[token];
            if (head < rope.heads + rope.kv_heads && early_pos >= 0 && early_pos < rope.table_len) {
                const float* cs = rope.cos_sin + (size_t)early_pos * rope.head_dim;
                early_cos = cs[d]; early_sin = cs[rope.head_dim / 2 + d];
            }
            if (head >= rope.heads && rope.slot_of) early_slot = rope.slot_of[token];
            if (p.bias) { early_bias_lo = __bfloat162float(p.bias[row0 + r]); early_bias_hi = __bfloat162float(p.bias[row8 + r]); }
        }
    }
    grid_dependency_wait();
    grid_dependents_go();
    // x: token 8 n + g, the same 16 bytes of k as this lane's weights (tokens beyond T read as zero);
    // every block reads the same few KB, which stay in L1 / L2
    const bf16* x_of[TT];
#pragma unroll
    for (int n = 0; n < TT; ++n) x_of[n] = (8 * n + g < p.T) ? p.x + (size_t)(8 * n + g) * p.ldx + 8 * t : nullptr;

    float acc[TT][4];
#pragma unroll
    for (int n = 0; n < TT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    int slot = 0;
    auto multiply = [&](const uint4 (&b)[TT], int c) {              // chunk c of the weights (this slot) times the tokens' chunk
        cp_async_wait<SK_AHEAD - 1>();                            // the oldest group - this slot - has landed
        const uint4 a_lo = *reinterpret_cast<const uint4*>(mine + slot * 1024);
        const uint4 a_hi = *reinterpret_cast<const uint4*>(mine + slot * 1024 + 512);
#pragma unroll
        for (int n = 0; n < TT; ++n) {
            mma_16x8x16(acc[n], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b[n].x, b[n].y);
            mma_16x8x16(acc[n], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b[n].z, b[n].w);
        }
        ask(slot, c + SK_WARPS * SK_AHEAD);                       // refill what has just been used
        slot = slot + 1 == SK_AHEAD ? 0 : slot + 1;
    };
    // the x values of four of the warp's chunks are asked for together: a trip to L2 per four chunks
    // instead of one per chunk (two chunks with more than 8 tokens: the registers of four would
    // cost the second block that an SM holds)
    constexpr int X_AHEAD = TT == 1 ? 4 : 2;
    for (int c0 = warp; c0 < chunks; c0 += X_AHEAD * SK_WARPS) {
        uint4 b[X_AHEAD][TT];
#pragma unroll
        for (int j = 0; j < X_AHEAD; ++j) {
            const int c = c0 + j * SK_WARPS;
#pragma unroll
            for (int n = 0; n < TT; ++n)
                b[j][n] = (c < chunks && x_of[n]) ? *reinterpret_cast<const uint4*>(x_of[n] + c * SK_CHUNK) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < X_AHEAD; ++j) {
            const int c = c0 + j * SK_WARPS;
            if (c < chunks) multiply(b[j], c);
        }
    }
    cp_async_wait<0>();
    // acc[n]: rows g (0, 1) and g + 8 (2, 3), tokens 8 n + 2 t and 8 n + 2 t + 1
#pragma unroll
    for (int n = 0; n < TT; ++n) {
        float* mine = red + ((size_t)warp * SK_ROWS) * TP + 8 * n + 2 * t;
        mine[(size_t)g * TP] = acc[n][0];
        mine[(size_t)g * TP + 1] = acc[n][1];
        mine[(size_t)(g + 8) * TP] = acc[n][2];
        mine[(size_t)(g + 8) * TP + 1] = acc[n][3];
    }
    __syncthreads();
    if constexpr (ROPE) {
        const int half = rope.head_dim / 2;
        const int per_head = rope.head_dim / 16;
        const int head = blockIdx.x / per_head, d0 = (blockIdx.x - head * per_head) * 8;
        for (int e = threadIdx.x; e < 8 * TP; e += blockDim.x) {
            const int token = e >> 3, r = e & 7;                  // consecutive threads: consecutive pairs of a token
            if (token >= p.T) continue;
            float lo = 0.f, hi = 0.f;
#pragma unroll
            for (int w = 0; w < SK_WARPS; ++w) {
                lo += red[((size_t)w * SK_ROWS + r) * TP + token];
                hi += red[((size_t)w * SK_ROWS + r + 8) * TP + token];
            }
            lo += early_bias_lo; hi += early_bias_hi;             // (e is this thread's own pair: see above)
            // the unfused path stores the product as bfloat16 before it rotates: the same rounding here
            lo = __bfloat162float(__float2bfloat16_rn(lo));
            hi = __bfloat162float(__float2bfloat16_rn(hi));
            const int d = d0 + r;
            if (head < rope.heads + rope.kv_heads) {              // a query or key head: rotate
                float c = early_cos, sn = early_sin;
                if (early_pos < 0 || early_pos >= rope.table_len) {     // refused: as position 0, and the step fails
                    atomicExch(rope.error, 2);
                    c = rope.cos_sin[d]; sn = rope.cos_sin[half + d];
                }
                const float a = lo * c - hi * sn, b = hi * c + lo * sn;
                lo = a; hi = b;
            }
            bf16* dst;
            if (head < rope.heads) {
                dst = reinterpret_cast<bf16*>(p.y) + (size_t)token * p.ldy + head * rope.head_dim;
            } else {
                const int slot = early_slot;
                if (slot < 0) continue;
                const long long page = slot / rope.page_size;
                const int offset = slot - (int)page * rope.page_size;
                const bool is_k = head < rope.heads + rope.kv_heads;
                const int kvh = head - rope.heads - (is_k ? 0 : rope.kv_heads);
                dst = (is_k ? rope.k_pages : rope.v_pages) + page * rope.page_stride +
                      ((size_t)kvh * rope.page_size + offset) * rope.head_dim;
            }
            dst[d] = __float2bfloat16_rn(lo);
            dst[half + d] = __float2bfloat16_rn(hi);
        }
    } else {
    for (int e = threadIdx.x; e < SK_ROWS * TP; e += blockDim.x) {
        const int token = e / SK_ROWS, r = e - token * SK_ROWS;   // consecutive threads: consecutive outputs of a token
        const int n = row0 + r;
        if (token >= p.T || n >= p.N) continue;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) sum += red[((size_t)w * SK_ROWS + r) * TP + token];
        if (p.bias) sum += __bfloat162float(p.bias[n]);
        if (p.out_f32) reinterpret_cast<float*>(p.y)[(size_t)token * p.ldy + n] = sum;
        else reinterpret_cast<bf16*>(p.y)[(size_t)token * p.ldy + n] = __float2bfloat16_rn(sum);
    }
    }
}

template <int TT, bool ROPE>
static int launch_skinny(const SkinnyParams& p, const SkinnyRope& rope, cudaStream_t stream) {
    constexpr size_t smem = (size_t)SK_WARPS * SK_AHEAD * 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<TT, ROPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return launch_dependent(gemm_skinny_kernel<TT, ROPE>, dim3((p.N + SK_ROWS - 1) / SK_ROWS), dim3(32 * SK_WARPS), smem, stream, p, rope);
}

}  // namespace fsie

using namespace fsie;

extern "C" {

// y[T, N] = x[T, K] * w^T (+ bias); T <= 16, K a multiple of 32, rows of x and w on 16-byte boundaries.
int fsie_gemm_skinny(const void* w, const void* x, long long ldx, void* y, long long ldy, const void* bias,
                     int T, int N, int K, int out_f32, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (T > 16 || K <= 0 || K % SK_CHUNK != 0 || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(w) & 15) ||
        (reinterpret_cast<uintptr_t>(x) & 15))
        return ERR_BAD_ARGUMENT;
    SkinnyParams p;
    p.w = (const bf16*)w; p.x = (const bf16*)x; p.ldx = ldx; p.y = y; p.ldy = ldy; p.bias = (const bf16*)bias;
    p.T = T; p.N = N; p.K = K; p.out_f32 = out_f32;
    SkinnyRope none = {};
    return T <= 8 ? launch_skinny<1, false>(p, none, stream) : launch_skinny<2, false>(p, none, stream);
}

// The q, k, v product fused with the rotation and the cache write (see SkinnyRope): w [(heads +
// 2 kv_heads) * head_dim, K]; rotated queries to q_out[T, ldq] (bfloat16), keys and values to
// slot_of[t] of the pages unless that is negative or k_pages is null.  head_dim a multiple of 16;
// the whole head is rotated (cos_sin has head_dim floats per position: cos | sin).
int fsie_gemm_skinny_qkv_rope(const void* w, const void* x, long long ldx, void* q_out, long long ldq, const void* bias,
                              int T, int K, const int* positions, const float* cos_sin, int table_len,
                              const int* slot_of, void* k_pages, void* v_pages, long long page_stride, int page_size,
                              int heads, int kv_heads, int head_dim, int* error, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (T > 16 || K <= 0 || K % SK_CHUNK != 0 || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(w) & 15) ||
        (reinterpret_cast<uintptr_t>(x) & 15) || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || head_dim % 16 != 0 ||
        !positions || !cos_sin || !error || page_size <= 0)
        return ERR_BAD_ARGUMENT;
    SkinnyParams p;
    p.w = (const bf16*)w; p.x = (const bf16*)x; p.ldx = ldx; p.y = q_out; p.ldy = ldq; p.bias = (const bf16*)bias;
    p.T = T; p.N = (heads + 2 * kv_heads) * head_dim; p.K = K; p.out_f32 = 0;
    SkinnyRope rope;
    rope.positions = positions; rope.cos_sin = cos_sin; rope.table_len = table_len;
    rope.slot_of = k_pages ? slot_of : nullptr; rope.k_pages = (bf16*)k_pages; rope.v_pages = (bf16*)v_pages;
    rope.page_stride = page_stride; rope.page_size = page_size;
    rope.heads = heads; rope.kv_heads = kv_heads; rope.head_dim = head_dim; rope.error = error;
    return T <= 8 ? launch_skinny<1, true>(p, rope, stream) : launch_skinny<2, true>(p, rope, stream);
}

}  // extern "C"
