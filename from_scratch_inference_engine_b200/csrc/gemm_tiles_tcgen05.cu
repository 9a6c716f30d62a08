// Matrix product for steps with many tokens (prompts and their portions):
// y[M, N] = x[M, K] * w[N, K]^T, bfloat16 operands, 32-bit accumulation on the 5th-generation
// tensor cores, with the bias add or the SwiGLU activation applied to the accumulator before
// anything is written.
//
// A persistent grid of one block per SM walks over 256 x 256 output tiles.  Per k-block of 64
// one thread issues four TMA boxes (two of x, two of w; 128 rows x 128 bytes each, 128-byte
// swizzle) into a ring of three 64 KB stages; one thread issues eight tcgen05.mma of
// 128 x 256 x 16 - the two row halves of the tile share the w boxes in shared memory - into
// two accumulators that fill all 512 columns of tensor memory; eight warps read a finished
// tile back (tcgen05.ld), apply the epilogue and store rows while the copy engine already
// fetches the next tile's first stages.
//
// Tiles are numbered row-tile fastest, so blocks that run at the same time share a few w
// tiles and all of x in L2, and w is read from HBM once.
//
// SwiGLU: w holds the gate rows and then the up rows; a tile takes 128 of each (the second
// w box starts at the up rows) and writes 128 columns of silu(gate) * up.
//
// Rows of x beyond M and rows of w beyond its end are zero-filled by TMA and never stored.
// Every wait on an mbarrier is bounded: when it runs out the kernel records where in
// *error, waits for the copies it started, frees its tensor memory and returns.
#include "common.cuh"
#include "tma.cuh"
#include <math.h>
#include <string.h>

namespace fsie {

constexpr int HALF = 128;                    // rows of one MMA (UMMA M) and of one TMA box
constexpr int TILE = 256;                    // tile rows and columns
constexpr int BK = 64;                       // k elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 3;
constexpr uint32_t BOX_BYTES = HALF * BK * 2;            // 16 KB
constexpr uint32_t STAGE_BYTES = 4 * BOX_BYTES;          // x rows 0-127, x rows 128-255, w 0-127, w 128-255
constexpr uint32_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES;
constexpr int EPILOGUE_WARPS = 8;
constexpr int THREADS = 64 + 32 * EPILOGUE_WARPS;
constexpr uint32_t TMEM_COLS = 512;

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1 };
enum { ERR_TMA_WAIT = 21, ERR_MMA_WAIT = 22, ERR_ACC_WAIT = 23, ERR_EPILOGUE_WAIT = 24 };

struct TileGemmParams {
    void* y; long long ldy;         // [M, ldy] bf16 or float
    const bf16* bias;               // [N] or null
    int M, N, K;                    // N = output features (SwiGLU: the intermediate size)
    int up_row0;                    // SwiGLU: row of w where the up rows start
    int m_tiles, n_tiles;
    int out_f32;
    int* error;
};

// Shared-memory matrix descriptor of a K-major tile in the 128-byte swizzle: rows of 128
// bytes, groups of 8 rows 1,024 bytes apart (stride byte offset), version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr(tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)(1) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor: D float, A and B bfloat16, both K-major, M x N.
__device__ __forceinline__ uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// 32 consecutive accumulator columns of this warp's 32 lanes: v[j] = D[lane, column + j]
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Stores 32 consecutive outputs of one row, columns n .. n + 31 as far as they lie below N.
__device__ __forceinline__ void store_row_chunk(const TileGemmParams& p, int row, int n, const float* v, bool vector_ok) {
    if (row >= p.M) return;
    if (p.out_f32) {
        float* dst = reinterpret_cast<float*>(p.y) + (size_t)row * p.ldy + n;
        if (vector_ok && n + 32 <= p.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (n + j < p.N) dst[j] = v[j];
        }
    } else {
        bf16* dst = reinterpret_cast<bf16*>(p.y) + (size_t)row * p.ldy + n;
        if (vector_ok && n + 32 <= p.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                uint4 w;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]), h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                w.x = *reinterpret_cast<uint32_t*>(&h0); w.y = *reinterpret_cast<uint32_t*>(&h1);
                w.z = *reinterpret_cast<uint32_t*>(&h2); w.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(dst + j) = w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (n + j < p.N) dst[j] = __float2bfloat16_rn(v[j]);
        }
    }
}

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tiles_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                  const TileGemmParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full, acc_empty;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (p.K + BK - 1) / BK;
    const int total_tiles = p.m_tiles * p.n_tiles;
    constexpr int TILE_COLS = EPI == EPI_SWIGLU ? TILE / 2 : TILE;      // output columns per tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, EPILOGUE_WARPS);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {        // one warp allocates all of tensor memory: two 128 x 256 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_slot;
    // x is the output of the kernel before this one; the kernel after this one may set up now
    grid_dependency_wait();
    grid_dependents_go();

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ TMA producer
        int it = 0, issued = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int m0 = (tile % p.m_tiles) * TILE, n0 = (tile / p.m_tiles) * TILE_COLS;
            const bool two_halves = p.M - m0 > HALF;
            const int w1_row = EPI == EPI_SWIGLU ? p.up_row0 + n0 : n0 + HALF;
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1)) {
                    atomicExch(p.error, ERR_TMA_WAIT); atomicExch(&abort_flag, 1);
                }
                if (*(volatile int*)&abort_flag) { ok = false; break; }
                unsigned char* stage = smem + s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], two_halves ? 4 * BOX_BYTES : 3 * BOX_BYTES);
                tma_load_2d(stage, &map_x, kb * BK, m0, &full_bar[s]);
                if (two_halves) tma_load_2d(stage + BOX_BYTES, &map_x, kb * BK, m0 + HALF, &full_bar[s]);
                tma_load_2d(stage + 2 * BOX_BYTES, &map_w, kb * BK, n0, &full_bar[s]);
                tma_load_2d(stage + 3 * BOX_BYTES, &map_w, kb * BK, w1_row, &full_bar[s]);
                issued = it + 1;
            }
        }
        if (!ok) {
            // giving up: let the copies already issued land before the block's memory is released
            for (int j = max(0, issued - STAGES); j < issued; ++j) mbar_wait(&full_bar[j % STAGES], (j / STAGES) & 1);
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------ MMA issuer
        const uint32_t idesc = umma_idesc(HALF, TILE);
        int it = 0, local_tile = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local_tile) {
            const int m0 = (tile % p.m_tiles) * TILE;
            const bool two_halves = p.M - m0 > HALF;
            if (local_tile > 0) {       // the epilogue warps have read the previous tile out of tensor memory
                if (!mbar_wait(&acc_empty, (local_tile - 1) & 1)) {
                    atomicExch(p.error, ERR_ACC_WAIT); atomicExch(&abort_flag, 1); ok = false; break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                const int s = it % STAGES;
                if (*(volatile int*)&abort_flag) { ok = false; break; }
                if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) {
                    atomicExch(p.error, ERR_MMA_WAIT); atomicExch(&abort_flag, 1); ok = false; break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned char* stage = smem + s * STAGE_BYTES;
                const uint64_t a0 = umma_desc(stage), a1 = umma_desc(stage + BOX_BYTES), b = umma_desc(stage + 2 * BOX_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    // 16 elements further along k: 32 bytes inside the swizzled row (address field in 16-byte units)
                    const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                    umma_bf16(tmem, a0 + 2 * k, b + 2 * k, idesc, accumulate);
                    if (two_halves) umma_bf16(tmem + TILE, a1 + 2 * k, b + 2 * k, idesc, accumulate);
                }
                umma_commit(&empty_bar[s]);          // the stage is free once these MMAs have read it
            }
            umma_commit(&acc_full);                  // the tile's accumulators are complete
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;                // the tensor-memory lanes this warp may read
        const int column_half = (warp - 2) >> 2;     // which half of the tile's output columns
        const bool vector_ok = (p.ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0);
        int local_tile = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local_tile) {
            const int m0 = (tile % p.m_tiles) * TILE, n0 = (tile / p.m_tiles) * TILE_COLS;
            const bool two_halves = p.M - m0 > HALF;
            if (*(volatile int*)&abort_flag) break;
            if (!mbar_wait(&acc_full, local_tile & 1)) {
                atomicExch(p.error, ERR_EPILOGUE_WAIT); atomicExch(&abort_flag, 1); break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int h = 0; h < (two_halves ? 2 : 1); ++h) {
                const int row = m0 + h * HALF + quarter * 32 + lane;
                const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16) + h * TILE;
                if (EPI == EPI_SWIGLU) {
#pragma unroll 1
                    for (int c = 0; c < 2; ++c) {
                        const int col = column_half * 64 + c * 32, n = n0 + col;
                        if (n >= p.N) continue;
                        float g[32], u[32];
                        tmem_load_32(trow + col, g);
                        tmem_load_32(trow + HALF + col, u);
                        tmem_load_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            // gate and up are rounded to bfloat16 before the activation, as the
                            // unfused path stores them in between
                            const float gj = __bfloat162float(__float2bfloat16_rn(g[j]));
                            const float uj = __bfloat162float(__float2bfloat16_rn(u[j]));
                            g[j] = (gj / (1.0f + expf(-gj))) * uj;
                        }
                        store_row_chunk(p, row, n, g, vector_ok);
                    }
                } else {
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        const int col = column_half * 128 + c * 32, n = n0 + col;
                        if (n >= p.N) continue;
                        float v[32];
                        tmem_load_32(trow + col, v);
                        tmem_load_wait();
                        if (p.bias) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) if (n + j < p.N) v[j] += __bfloat162float(p.bias[n + j]);
                        }
                        store_row_chunk(p, row, n, v, vector_ok);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty);
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// bf16 matrix [rows, cols] with `ld` elements between rows; boxes of 128 rows x 64 columns, 128-byte swizzle
static int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)HALF};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                               elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? 0 : ERR_BAD_ARGUMENT;
}

template <int EPI>
static int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const TileGemmParams& p, int blocks,
                  cudaStream_t stream) {
    auto kernel = gemm_tiles_kernel<EPI>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return launch_dependent(kernel, dim3(blocks), dim3(THREADS), SMEM_BYTES, stream, map_w, map_x, p);
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_gemm_tiles_map_bytes() { return (int)sizeof(CUtensorMap); }

// Describe a bf16 weight matrix w[rows, K] (K contiguous) for the kernel below.
int fsie_gemm_tiles_weight_map(void* map_out, const void* w, long long rows, long long K) {
    if (K % 8 != 0 || (reinterpret_cast<uintptr_t>(w) & 15)) return ERR_BAD_ARGUMENT;
    CUtensorMap map;
    const int rc = make_map(&map, w, rows, K, K);
    if (rc == 0) memcpy(map_out, &map, sizeof(map));
    return rc;
}

// y[M, N] = x[M, K] * w^T (+ bias), or for swiglu y[M, N] = silu(x w_gate^T) * (x w_up^T) with
// w = [gate rows (N); up rows (N)].  `blocks` is the size of the persistent grid (the number
// of SMs; fewer when there are fewer tiles).
int fsie_gemm_tiles(const void* weight_map, const void* x, long long ldx, void* y, long long ldy, const void* bias,
                    int M, int N, int K, int swiglu, int out_f32, int blocks, int* error, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || blocks <= 0 || (swiglu && out_f32))
        return ERR_BAD_ARGUMENT;
    CUtensorMap map_w, map_x;
    memcpy(&map_w, weight_map, sizeof(map_w));
    int rc = make_map(&map_x, x, M, K, ldx);
    if (rc != 0) return rc;
    TileGemmParams p;
    p.y = y; p.ldy = ldy; p.bias = (const bf16*)bias; p.M = M; p.N = N; p.K = K;
    p.up_row0 = N; p.out_f32 = out_f32; p.error = error;
    p.m_tiles = (M + TILE - 1) / TILE;
    p.n_tiles = swiglu ? (N + TILE / 2 - 1) / (TILE / 2) : (N + TILE - 1) / TILE;
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    if (tiles < blocks) blocks = (int)tiles;
    return swiglu ? launch<EPI_SWIGLU>(map_w, map_x, p, blocks, stream) : launch<EPI_PLAIN>(map_w, map_x, p, blocks, stream);
}

}  // extern "C"
