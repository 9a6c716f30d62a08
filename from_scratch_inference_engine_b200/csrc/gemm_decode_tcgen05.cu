// Matrix product for steps with few tokens (decode): y[T, N] = x[T, K] * w[N, K]^T with
// T <= 64, bfloat16 operands, 32-bit accumulation, on the 5th-generation tensor cores.
//
// With so few tokens the product is bound by streaming w once from HBM, so the roles are
// swapped: a block owns 128 rows of w as the M side of a 128 x TN x 16 tcgen05.mma
// (TN = tokens padded to 16, 32 or 64), the tokens are the N side, and the accumulator
// D[128 weight rows, TN tokens] lives in tensor memory.  One thread issues TMA loads of the
// 128 x 64 weight tile and the TN x 64 activation tile of each k-block into a ring of
// shared-memory stages (128-byte swizzle, mbarrier full/empty pairs), one thread issues
// the MMAs, four warps read the accumulator back (tcgen05.ld) for the epilogue.
//
// When N / 128 blocks are too few to fill the GPU the k range is split over the blocks of
// a thread-block cluster; their partial sums meet through distributed shared memory and
// are added in rank order (no atomics, the same bits on every run).
//
// Epilogues: bias add; SwiGLU (w holds gate rows then up rows, a block takes 64 of each
// and writes silu(gate) * up); 32-bit output for logits.
//
// Every wait on an mbarrier is bounded: when it runs out the kernel records where in
// *error, drains what it started, frees its tensor memory and returns.
#include "common.cuh"
#include "tma.cuh"
#include <cooperative_groups.h>
#include <math.h>
#include <string.h>

namespace fsie {
namespace cg = cooperative_groups;

constexpr int BM = 128;            // weight rows per block (UMMA M)
constexpr int BK = 64;             // k elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1 };
enum { ERR_TMA_WAIT = 11, ERR_MMA_WAIT = 12, ERR_EPILOGUE_WAIT = 13 };

struct GemmParams {
    void* y; int ldy;               // [T, ldy] bf16 or float
    const bf16* bias;               // [N] or null
    int T, N, K;                    // N = output features (SwiGLU: intermediate size)
    int up_row0;                    // SwiGLU: row of w where the up rows start
    int kblocks_per_split;
    int out_f32;
    int* error;
};

// Shared-memory matrix descriptor of a K-major tile in the 128-byte swizzle: rows of 128
// bytes, groups of 8 rows 1,024 bytes apart (stride byte offset), version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr(tile) & 0x3FFFF) >> 4);          // start address
    d |= (uint64_t)(1) << 16;                                   // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                           // stride byte offset
    d |= (uint64_t)1 << 46;                                     // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                                     // SWIZZLE_128B
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

template <int TN> struct Layout {
    static constexpr int STAGES = 4;                             // ~72-97 KB: two or three blocks per SM overlap
                                                                 // one block's epilogue with the others' streaming
    static constexpr uint32_t A_BYTES = BM * BK * 2;             // 16 KB
    static constexpr uint32_t B_BYTES = TN * BK * 2;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t RED_LD = TN + 1;                   // padded row of the exchange area
    static constexpr uint32_t RED_BYTES = BM * RED_LD * 4;
    static constexpr uint32_t PIPE_BYTES = STAGES * STAGE_BYTES;
    static constexpr uint32_t SMEM = 1024 + (PIPE_BYTES > RED_BYTES ? PIPE_BYTES : RED_BYTES);   // + alignment slack
    static constexpr uint32_t TMEM_COLS = TN < 32 ? 32 : TN;
};

// grid (N tiles, splits); with splits > 1 the blocks of one tile form a cluster along y.
template <int TN, int EPI>
__global__ void __launch_bounds__(192)
gemm_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const GemmParams p) {
    using L = Layout<TN>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full_bar[L::STAGES], empty_bar[L::STAGES], acc_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
    const int total_kblocks = (p.K + BK - 1) / BK;
    const int kb0 = min(total_kblocks, split * p.kblocks_per_split);
    const int kb1 = min(total_kblocks, kb0 + p.kblocks_per_split);
    const int n0 = EPI == EPI_SWIGLU ? tile * (BM / 2) : tile * BM;

    auto load_weights = [&](int kb, int s) {
        unsigned char* a = smem + s * L::STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);     // the activation tile's bytes are counted here too
        if (EPI == EPI_SWIGLU) {                      // 64 gate rows, then the 64 up rows of the same outputs
            tma_load_2d(a, &map_w, kb * BK, n0, &full_bar[s]);
            tma_load_2d(a + L::A_BYTES / 2, &map_w, kb * BK, p.up_row0 + n0, &full_bar[s]);
        } else {
            tma_load_2d(a, &map_w, kb * BK, n0, &full_bar[s]);
        }
    };
    auto load_activations = [&](int kb, int s) {
        tma_load_2d(smem + s * L::STAGE_BYTES + L::A_BYTES, &map_x, kb * BK, 0, &full_bar[s]);
    };
    auto load_stage = [&](int kb, int s) { load_weights(kb, s); load_activations(kb, s); };
    if (threadIdx.x == 0) {
        for (int s = 0; s < L::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // The producer fills the ring at once; tensor memory is allocated meanwhile.  Weights do
        // not depend on the kernel before this one: under programmatic dependent launch they are
        // fetched while that kernel still runs; its output (the activations) is read only after
        // griddepcontrol.wait.
        for (int it = 0; it < L::STAGES && kb0 + it < kb1; ++it) load_weights(kb0 + it, it);
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int it = 0; it < L::STAGES && kb0 + it < kb1; ++it) load_activations(kb0 + it, it);
    }
    if (warp == 1) {        // one warp allocates the accumulator's columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)), "r"(L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = tmem_base_slot;
    // every thread: nothing of the previous kernel is touched before it has completed (thread 0
    // waited above already); and the kernel after this one may start its own set-up now
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ TMA producer
        // (its first STAGES loads were issued before the block-wide barrier above)
        int issued = min(kb1 - kb0, L::STAGES);
        for (int kb = kb0 + L::STAGES; kb < kb1; ++kb) {
            const int it = kb - kb0, s = it % L::STAGES;
            if (!mbar_wait(&empty_bar[s], ((it / L::STAGES) - 1) & 1)) {
                atomicExch(p.error, ERR_TMA_WAIT); atomicExch(&abort_flag, 1); break;
            }
            if (*(volatile int*)&abort_flag) break;
            issued = it + 1;
            load_stage(kb, s);
        }
        if (*(volatile int*)&abort_flag) {
            // giving up: let the copies already issued land before the block's memory is released
            for (int it = max(0, issued - L::STAGES); it < issued; ++it)
                mbar_wait(&full_bar[it % L::STAGES], (it / L::STAGES) & 1);
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------ MMA issuer
        const uint32_t idesc = umma_idesc(BM, TN);
        bool ok = true;
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
            const int it = kb - kb0, s = it % L::STAGES;
            if (*(volatile int*)&abort_flag) break;
            if (!mbar_wait(&full_bar[s], (it / L::STAGES) & 1)) {
                atomicExch(p.error, ERR_MMA_WAIT); atomicExch(&abort_flag, 1); ok = false; break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned char* a = smem + s * L::STAGE_BYTES;
            const uint64_t a_desc = umma_desc(a), b_desc = umma_desc(a + L::A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
                // 16 elements further along k: 32 bytes inside the swizzled row (address field is in 16-byte units)
                umma_bf16(tmem_acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(&empty_bar[s]);              // the stage is free once these MMAs have read it
        }
        umma_commit(&acc_bar);                       // the accumulator is complete (or nothing was issued)
    }

    // ---------------------------------------------------------------- epilogue
    float* red = reinterpret_cast<float*>(smem);     // [BM][RED_LD], reuses the pipeline's memory
    if (warp >= 2) {
        const int quarter = warp & 3;                // the tensor-memory lanes this warp may read
        const int row = quarter * 32 + lane;         // weight row inside the tile = accumulator lane
        bool ok = kb1 > kb0 ? mbar_wait(&acc_bar, 0) : true;
        if (!ok) { atomicExch(p.error, ERR_EPILOGUE_WAIT); atomicExch(&abort_flag, 1); }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float v[TN];
        if (ok && kb1 > kb0) {
#pragma unroll
            for (int c = 0; c < TN; c += 16) {
                uint32_t r[16];
                const uint32_t taddr = tmem_acc + ((uint32_t)(quarter * 32) << 16) + c;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                               "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                             : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) v[c + j] = __uint_as_float(r[j]);
            }
        } else {
#pragma unroll
            for (int c = 0; c < TN; ++c) v[c] = 0.f;
        }
        // all MMAs have completed (acc_bar), so the stages are no longer read: reuse them
#pragma unroll
        for (int c = 0; c < TN; ++c) red[row * L::RED_LD + c] = v[c];
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(L::TMEM_COLS) : "memory");
    }

    // ---- add the splits' partial sums in rank order, apply the epilogue, store
    int rank = 0;
    if (splits > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        rank = (int)cluster.block_rank();
    }
    constexpr int OUT_ROWS = EPI == EPI_SWIGLU ? BM / 2 : BM;     // outputs per tile
    const int rows_per_rank = OUT_ROWS / splits;                  // splits divides 64
    const int r_begin = rank * rows_per_rank;
    for (int e = threadIdx.x; e < rows_per_rank * TN; e += blockDim.x) {
        const int r = r_begin + e % rows_per_rank, t = e / rows_per_rank;
        const int n = n0 + r;
        if (t >= p.T || n >= p.N) continue;
        float acc = 0.f, acc_up = 0.f;
        if (splits > 1) {
            cg::cluster_group cluster = cg::this_cluster();
            for (int q = 0; q < splits; ++q) {
                const float* theirs = cluster.map_shared_rank(red, q);
                acc += theirs[r * L::RED_LD + t];
                if (EPI == EPI_SWIGLU) acc_up += theirs[(r + BM / 2) * L::RED_LD + t];
            }
        } else {
            acc = red[r * L::RED_LD + t];
            if (EPI == EPI_SWIGLU) acc_up = red[(r + BM / 2) * L::RED_LD + t];
        }
        float out;
        if (EPI == EPI_SWIGLU) {
            // the library path rounds gate and up to bfloat16 before the activation; do the same
            const float g = __bfloat162float(__float2bfloat16_rn(acc));
            const float u = __bfloat162float(__float2bfloat16_rn(acc_up));
            out = (g / (1.0f + expf(-g))) * u;
        } else {
            out = acc + (p.bias ? __bfloat162float(p.bias[n]) : 0.f);
        }
        if (p.out_f32) reinterpret_cast<float*>(p.y)[(size_t)t * p.ldy + n] = out;
        else reinterpret_cast<bf16*>(p.y)[(size_t)t * p.ldy + n] = __float2bfloat16_rn(out);
    }
    if (splits > 1) cg::this_cluster().sync();        // nobody leaves while its sums may be read
}

// bf16 matrix [rows, cols] with `ld` elements between rows; boxes of box_rows x 64 columns, 128-byte swizzle
static int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                               elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? 0 : ERR_BAD_ARGUMENT;
}

template <int TN, int EPI>
static int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmParams& p, int tiles, int splits,
                  cudaStream_t stream) {
    using L = Layout<TN>;
    auto kernel = gemm_decode_kernel<TN, EPI>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::SMEM);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(tiles, splits, 1);
    config.blockDim = dim3(192, 1, 1);
    config.dynamicSmemBytes = L::SMEM;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = splits;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: this kernel's set-up and first weight tiles may overlap the
    // tail of the kernel before it in the stream (it waits before touching that kernel's output)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&config, kernel, map_w, map_x, p);
}

}  // namespace fsie

using namespace fsie;

extern "C" {

// Bytes of a tensor map; the caller keeps one per weight matrix.
int fsie_tensor_map_bytes() { return (int)sizeof(CUtensorMap); }

// Describe a bf16 weight matrix w[rows, K] (K contiguous) for the kernel below.  box_rows is
// 128 for a plain product and 64 for SwiGLU (gate and up halves are fetched separately).
int fsie_gemm_decode_weight_map(void* map_out, const void* w, long long rows, long long K, int box_rows) {
    if (K % 8 != 0 || (box_rows != 128 && box_rows != 64)) return ERR_BAD_ARGUMENT;
    CUtensorMap map;
    const int rc = make_map(&map, w, rows, K, K, box_rows);
    if (rc == 0) memcpy(map_out, &map, sizeof(map));
    return rc;
}

// y[T, N] = x[T, K] * w^T (+ bias), or for swiglu y[T, N] = silu(x w_gate^T) * (x w_up^T) with
// w = [gate rows (N); up rows (N)].  T <= 64.  `splits` (1, 2, 4 or 8) cuts K over a cluster.
int fsie_gemm_decode(const void* weight_map, const void* x, int ldx, void* y, int ldy, const void* bias,
                     int T, int N, int K, int swiglu, int out_f32, int splits, int* error, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (T > 64 || K <= 0 || K % 8 != 0 || ldx % 8 != 0 || (splits != 1 && splits != 2 && splits != 4 && splits != 8))
        return ERR_BAD_ARGUMENT;
    const int TN = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    CUtensorMap map_w, map_x;
    memcpy(&map_w, weight_map, sizeof(map_w));
    int rc = make_map(&map_x, x, T, K, ldx, TN);
    if (rc != 0) return rc;
    GemmParams p;
    p.y = y; p.ldy = ldy; p.bias = (const bf16*)bias; p.T = T; p.N = N; p.K = K;
    p.up_row0 = N; p.out_f32 = out_f32; p.error = error;
    const int total_kblocks = (K + BK - 1) / BK;
    p.kblocks_per_split = (total_kblocks + splits - 1) / splits;
    const int tiles = swiglu ? (N + BM / 2 - 1) / (BM / 2) : (N + BM - 1) / BM;
#define FSIE_GEMM(TNV)                                                                             \
    (swiglu ? launch<TNV, EPI_SWIGLU>(map_w, map_x, p, tiles, splits, stream)                      \
            : launch<TNV, EPI_PLAIN>(map_w, map_x, p, tiles, splits, stream))
    if (TN == 16) rc = FSIE_GEMM(16);
    else if (TN == 32) rc = FSIE_GEMM(32);
    else rc = FSIE_GEMM(64);
#undef FSIE_GEMM
    return rc;
}

}  // extern "C"
