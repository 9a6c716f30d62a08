// Matrix product for steps with many tokens (prompts and their portions):
// y[M, N] = x[M, K] * w[N, K]^T, bfloat16 operands, 32-bit accumulation on the 5th-generation
// tensor cores, with the bias add or the SwiGLU activation applied to the accumulator before
// anything is written.
//
// Two blocks on neighbouring SMs (a cluster of two) share every 256 x 256 output tile: each
// loads 128 rows of x and 128 rows of w per k-block of 64 (two TMA boxes of 16 KB into a ring
// of six 32 KB stages), one thread of the first block issues tcgen05.mma with cta_group::2 -
// 256 x 256 x 16 over both blocks' shared memory - and each block keeps its 128 rows of the
// result in its own tensor memory.  Halving the bytes each SM has to fetch per MMA is what
// lets the ring run far enough ahead of the tensor cores to hide the latency of L2.
// Tensor memory holds two accumulators per block (2 x 256 columns), so the eight epilogue
// warps of a block read a finished tile back (tcgen05.ld), apply the epilogue and store rows
// while the next tile's MMAs already run into the other accumulator.
//
// A persistent grid of one pair per two SMs walks over the tiles, row-tile fastest, so pairs
// that run at the same time share a few w tiles and all of x in L2, and w is read from HBM once.
//
// Barriers: a stage's "full" barrier lives in the first block and counts the bytes of both
// blocks' boxes; "empty" and "accumulator full" are signalled in both blocks at once by a
// multicast tcgen05.commit; "accumulator empty" lives in the first block and takes arrivals
// from the epilogue warps of both.
//
// SwiGLU: w holds the gate rows and then the up rows; of a tile's 256 accumulator columns the
// first block supplies 128 gate rows and the second the 128 up rows of the same outputs, and
// the epilogue writes 128 columns of silu(gate) * up.
//
// Tiles that do not fill a last round of the pairs (112 tiles on 74 pairs leave 36 pairs idle for
// a whole tile's time) are shared out: after the full rounds, the k-blocks of the remaining tiles
// are numbered tile after tile and cut into equal shares, one per pair, so a pair's share may end
// one tile and begin the next.  A pair that has summed only part of a tile's k range leaves its
// 32-bit sums in a workspace; the pair that arrives last at the tile's counter (per 32 rows, no
// pair waits for another) adds the parts in the order of the shares - the same bits on every run -
// and runs the epilogue.
//
// Rows of x beyond M and rows of w beyond its end are zero-filled by TMA and never stored.
// Every wait on an mbarrier is bounded: when it runs out the kernel records where in
// *error, lets the copies it started land, frees its tensor memory and returns.
#include "common.cuh"
#include "tma.cuh"
#include <math.h>
#include <string.h>

namespace fsie {

constexpr int HALF = 128;                    // rows per block: of x (MMA M = 2 x 128) and of w (N = 2 x 128)
constexpr int TILE = 256;                    // tile rows and accumulator columns
constexpr int ATOM_K = 64;                   // k elements of one TMA box: 128 bytes, one swizzle row
constexpr int ATOMS = 2;                     // boxes along k per stage and operand
constexpr int BK = ATOM_K * ATOMS;           // k elements per stage
constexpr int UMMA_K = 16;
constexpr int STAGES = 6 / ATOMS;
constexpr uint32_t BOX_BYTES = HALF * ATOM_K * 2;        // 16 KB
constexpr uint32_t STAGE_BYTES = 2 * ATOMS * BOX_BYTES;  // this block's rows of x, then its rows of w
constexpr uint32_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 4 * 2 * (32 * 128);   // ring + two output boxes per epilogue warp
constexpr int EPILOGUE_WARPS = 4;                        // one per quarter of the tensor-memory lanes
constexpr uint32_t OUT_BOX_BYTES = 32 * 128;             // 32 rows x 64 outputs, staged for a TMA store
constexpr int THREADS = 64 + 32 * EPILOGUE_WARPS;
constexpr uint32_t TMEM_COLS = 512;                      // two accumulators of 256 columns
constexpr uint32_t FIRST_BLOCK_MASK = 0xFEFFFFFFu;       // clears the bit of a shared::cluster address that
                                                         // tells the second block of a pair from the first

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1 };
enum { ERR_TMA_WAIT = 21, ERR_MMA_WAIT = 22, ERR_ACC_WAIT = 23, ERR_EPILOGUE_WAIT = 24 };

struct TileGemmParams {
    void* y; long long ldy;         // [M, ldy] bf16 or float
    const bf16* bias;               // [N] or null
    int M, N, K;                    // N = output features (SwiGLU: the intermediate size)
    int up_row0;                    // SwiGLU: row of w where the up rows start
    int m_tiles, n_tiles;
    int out_f32;
    int tma_store;                  // y is written through map_y (bf16, rows on 16-byte boundaries)
    // sharing of the last, partial round (share_pairs = 0: every tile is summed by one pair)
    int full_rounds;                // rounds in which every pair takes a whole tile
    int shared_tiles;               // tiles after those rounds
    int share_pairs;                // pairs that take an equal share of their k-blocks
    int max_parts;                  // most pairs that share one tile
    float* workspace;               // [shared tile][part][block of the pair][128 rows][256 columns]
    int* counters;                  // [shared tile][block of the pair][quarter], zero between launches
    int* error;
};

// One piece of work of a pair: k-blocks [kb0, kb1) of a tile.  shared >= 0: the tile is the
// shared one of that index and this pair sums part `part` of `parts` of its k range.
struct WorkItem { int tile, kb0, kb1, shared, part, parts; };

__host__ __device__ __forceinline__ long long share_begin(long long units, int pairs, int j) { return units * j / pairs; }
// the pair whose share holds unit u
__host__ __device__ __forceinline__ int share_of(long long units, int pairs, long long u) {
    int j = (int)(u * pairs / units);
    while (j + 1 < pairs && share_begin(units, pairs, j + 1) <= u) ++j;
    while (j > 0 && share_begin(units, pairs, j) > u) --j;
    return j;
}
// The pair's i-th piece of work; false when it has no more.
__device__ __forceinline__ bool work_item(const TileGemmParams& p, int pair, int pairs, int kblocks, int total_tiles,
                                          int i, WorkItem& w) {
    w.kb0 = 0; w.kb1 = kblocks; w.shared = -1; w.part = 0; w.parts = 1;
    if (p.share_pairs == 0) {
        w.tile = pair + i * pairs;
        return w.tile < total_tiles;
    }
    // The shared tiles come first: what their parts cost beyond the sums (the workspace traffic,
    // the adding by whoever comes last) then runs in the epilogue warps under the MMAs of the
    // whole tiles that follow.
    int pieces = 0;
    long long u0 = 0, u1 = 0;
    const long long units = (long long)p.shared_tiles * kblocks;
    if (pair < p.share_pairs) {
        u0 = share_begin(units, p.share_pairs, pair); u1 = share_begin(units, p.share_pairs, pair + 1);
        if (u1 > u0) pieces = (int)((u1 - 1) / kblocks - u0 / kblocks) + 1;
    }
    if (i >= pieces) {
        const int round = i - pieces;
        w.tile = pair + round * pairs;
        return round < p.full_rounds;
    }
    const int r = (int)(u0 / kblocks) + i;
    const long long first = (long long)r * kblocks;
    w.tile = p.full_rounds * pairs + r;
    w.kb0 = (int)(u0 > first ? u0 - first : 0);
    w.kb1 = (int)(u1 - first < kblocks ? u1 - first : kblocks);
    if (w.kb0 > 0 || w.kb1 < kblocks) {
        const int lowest = share_of(units, p.share_pairs, first);
        w.shared = r;
        w.part = pair - lowest;
        w.parts = share_of(units, p.share_pairs, first + kblocks - 1) - lowest + 1;
    }
    return true;
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;\n barrier.cluster.wait.acquire;" ::: "memory");
}
// TMA box into this block's shared memory; its bytes are counted by the barrier at the same
// offset in the first block of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_addr(bar) & FIRST_BLOCK_MASK) : "memory");
}
// Arrival on the barrier at this offset in the first block of the pair.
__device__ __forceinline__ void mbar_arrive_first_block(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_addr(bar) & FIRST_BLOCK_MASK) : "memory");
}

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
// One MMA over the pair: A rows and B rows at these offsets in both blocks' shared memory,
// D at this address in both blocks' tensor memory.  Issued by the first block only.
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// When the MMAs issued so far have completed, arrive on the barrier at this offset in both blocks.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_addr(bar)), "h"((uint16_t)3) : "memory");
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
// the reverse: D[lane, column + j] = v[j]
__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr),
          "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

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
                  const __grid_constant__ CUtensorMap map_y, const TileGemmParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank();            // 0: the block that issues the MMAs
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int kblocks = (p.K + BK - 1) / BK;
    const int total_tiles = p.m_tiles * p.n_tiles;
    // Order of the tiles: bands of up to RASTER_M tiles of rows, inside a band the rows run
    // fastest.  The pairs of blocks work on consecutive tiles at the same time, so a wave of
    // them covers a roughly square patch of y and fetches as few rows of x and w as 74 tiles
    // can need - with more than 2,048 rows of x, walking all rows for each column of tiles
    // would read the whole of x once per two or three columns (for the down product that is
    // more than L2 holds, and the product becomes bound by HBM instead of the tensor cores).
    constexpr int RASTER_M = 8;
    auto tile_m = [&](int tile) {
        const int band = tile / (RASTER_M * p.n_tiles), first = band * RASTER_M;
        const int height = min(RASTER_M, p.m_tiles - first);
        return first + (tile - band * RASTER_M * p.n_tiles) % height;
    };
    auto tile_n = [&](int tile) {
        const int band = tile / (RASTER_M * p.n_tiles), first = band * RASTER_M;
        const int height = min(RASTER_M, p.m_tiles - first);
        return (tile - band * RASTER_M * p.n_tiles) / height;
    };
    constexpr int TILE_COLS = EPI == EPI_SWIGLU ? TILE / 2 : TILE;      // output columns per tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * EPILOGUE_WARPS); }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {        // the same warp of both blocks allocates all of tensor memory in both
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();     // the other block's barriers are initialised before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_slot;
    // x is the output of the kernel before this one; the kernel after this one may set up now
    grid_dependency_wait();
    grid_dependents_go();

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ TMA producer (both blocks)
        int it = 0, issued = 0;
        bool ok = true;
        auto w_row_of = [&](int tile) {
            const int n0 = tile_n(tile) * TILE_COLS;
            return EPI == EPI_SWIGLU ? (rank == 0 ? n0 : p.up_row0 + n0) : n0 + rank * HALF;
        };
        WorkItem work;
        for (int item = 0; ok && work_item(p, pair, pairs, kblocks, total_tiles, item, work); ++item) {
            const int tile = work.tile;
            const int m0 = tile_m(tile) * TILE + rank * HALF;
            const int w_row = w_row_of(tile);
            for (int kb = work.kb0; kb < work.kb1; ++kb, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1)) {
                    atomicExch(p.error, ERR_TMA_WAIT); atomicExch(&abort_flag, 1);
                }
                if (*(volatile int*)&abort_flag) { ok = false; break; }
                unsigned char* stage = smem + s * STAGE_BYTES;
                if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);       // both blocks' boxes
#pragma unroll
                for (int a = 0; a < ATOMS; ++a) {
                    tma_load_2d_pair(stage + a * BOX_BYTES, &map_x, kb * BK + a * ATOM_K, m0, &full_bar[s]);
                    tma_load_2d_pair(stage + (ATOMS + a) * BOX_BYTES, &map_w, kb * BK + a * ATOM_K, w_row, &full_bar[s]);
                }
                issued = it + 1;
            }
        }
        if (!ok) {
            // giving up: let the copies already issued land before the block's memory is released
            if (rank == 0) {
                for (int j = max(0, issued - STAGES); j < issued; ++j) mbar_wait(&full_bar[j % STAGES], (j / STAGES) & 1);
            } else {
                for (int i = 0; i < 1000; ++i) __nanosleep(1000);
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ------------------------------------------------------------ MMA issuer (first block)
        const uint32_t idesc = umma_idesc(TILE, TILE);
        int it = 0, local_tile = 0;
        bool ok = true;
        WorkItem work;
        for (; ok && work_item(p, pair, pairs, kblocks, total_tiles, local_tile, work); ++local_tile) {
            const int buf = local_tile & 1;
            if (local_tile >= 2) {      // both blocks' epilogue warps have read this accumulator's previous tile
                if (!mbar_wait(&acc_empty[buf], ((local_tile >> 1) - 1) & 1)) {
                    atomicExch(p.error, ERR_ACC_WAIT); atomicExch(&abort_flag, 1); ok = false; break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            for (int kb = work.kb0; kb < work.kb1; ++kb, ++it) {
                const int s = it % STAGES;
                if (*(volatile int*)&abort_flag) { ok = false; break; }
                if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) {
                    atomicExch(p.error, ERR_MMA_WAIT); atomicExch(&abort_flag, 1); ok = false; break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned char* stage = smem + s * STAGE_BYTES;
#pragma unroll
                for (int at = 0; at < ATOMS; ++at) {
                    const uint64_t a = umma_desc(stage + at * BOX_BYTES), b = umma_desc(stage + (ATOMS + at) * BOX_BYTES);
#pragma unroll
                    for (int k = 0; k < ATOM_K / UMMA_K; ++k) {
                        // 16 elements further along k: 32 bytes inside the swizzled row (address field in 16-byte units)
                        umma_bf16_pair(tmem + buf * TILE, a + 2 * k, b + 2 * k, idesc, (kb > work.kb0 || at > 0 || k > 0) ? 1u : 0u);
                    }
                }
                umma_commit_pair(&empty_bar[s]);     // the stage is free in both blocks once these MMAs have read it
            }
            if (ok) umma_commit_pair(&acc_full[buf]);        // the tile's accumulators are complete in both blocks
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue (both blocks)
        // A warp owns 32 rows of the block's 128.  It turns 32 accumulator columns at a time into
        // outputs; two such chunks fill a box of 32 rows x 128 bytes in shared memory (128-byte
        // swizzle, so that the lanes' 16-byte stores do not collide), which one TMA store writes to
        // y: whole lines, off the load/store path that stores of a row per lane would flood.
        const int quarter = warp & 3;                // the tensor-memory lanes this warp may read
        const bool vector_ok = (p.ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0);
        unsigned char* boxes = smem + STAGES * STAGE_BYTES + (warp - 2) * 2 * OUT_BOX_BYTES;
        int local_tile = 0, groups = 0;
        WorkItem work;
        for (; work_item(p, pair, pairs, kblocks, total_tiles, local_tile, work); ++local_tile) {
            const int tile = work.tile;
            const int buf = local_tile & 1;
            const int row0 = tile_m(tile) * TILE + rank * HALF + quarter * 32;
            const int n0 = tile_n(tile) * TILE_COLS;
            if (*(volatile int*)&abort_flag) break;
            if (!mbar_wait(&acc_full[buf], (local_tile >> 1) & 1)) {
                atomicExch(p.error, ERR_EPILOGUE_WAIT); atomicExch(&abort_flag, 1); break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16) + buf * TILE;
            // ---- a tile whose k range this pair has summed only in part
            // Workspace of one part and one warp: 8 chunks of 32 columns, a chunk as 8 x 32 lanes x 16
            // bytes, so that a warp's store (and the load of the same lane later) is one 512-byte run.
            constexpr size_t WARP_FLOATS = (size_t)32 * TILE, PART_FLOATS = (size_t)2 * HALF * TILE;
            if (work.shared >= 0) {
                float* warp_of_part0 = p.workspace + (size_t)work.shared * p.max_parts * PART_FLOATS +
                                       ((size_t)rank * EPILOGUE_WARPS + quarter) * WARP_FLOATS;
                float* mine = warp_of_part0 + (size_t)work.part * PART_FLOATS;
#pragma unroll 1
                for (int c = 0; c < TILE / 32; ++c) {
                    float v[32];
                    tmem_load_32(trow + c * 32, v);
                    tmem_load_wait();
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        __stcg(reinterpret_cast<float4*>(mine + c * 1024 + q * 128 + lane * 4),
                               make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
                }
                __threadfence();
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    int* counter = p.counters + (work.shared * 2 + rank) * EPILOGUE_WARPS + quarter;
                    last = atomicAdd(counter, 1) == work.parts - 1;
                    if (last) *counter = 0;          // for the next launch; nobody else comes in this one
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (!last) {                         // another pair will add the parts and store
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive_first_block(&acc_empty[buf]);
                    continue;
                }
                __threadfence();
                // Add the parts (four at most) into the accumulator in tensor memory, in the order of
                // the shares: this pair's own part comes from tensor memory, the others' are asked for
                // together.  The epilogue below then finds the whole sums where it always finds them.
#pragma unroll 1
                for (int c = 0; c < TILE / 32; ++c) {
                    float4 theirs[3][8];
#pragma unroll
                    for (int o = 0; o < 3; ++o) {
                        const int part = o < work.part ? o : o + 1;      // the o-th part that is not this pair's
                        if (part < work.parts) {
                            const float* src = warp_of_part0 + (size_t)part * PART_FLOATS + c * 1024 + lane * 4;
#pragma unroll
                            for (int q = 0; q < 8; ++q) theirs[o][q] = __ldcg(reinterpret_cast<const float4*>(src + q * 128));
                        }
                    }
                    float own[32], sum[32];
                    tmem_load_32(trow + c * 32, own);
                    tmem_load_wait();
#pragma unroll
                    for (int part = 0; part < 4; ++part) {
                        if (part >= work.parts) break;
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            float4 t;
                            if (part == work.part) t = make_float4(own[4 * q], own[4 * q + 1], own[4 * q + 2], own[4 * q + 3]);
                            else if (part < work.part) t = theirs[part < 3 ? part : 2][q];
                            else t = theirs[part > 0 ? part - 1 : 0][q];
                            if (part == 0) { sum[4 * q] = t.x; sum[4 * q + 1] = t.y; sum[4 * q + 2] = t.z; sum[4 * q + 3] = t.w; }
                            else { sum[4 * q] += t.x; sum[4 * q + 1] += t.y; sum[4 * q + 2] += t.z; sum[4 * q + 3] += t.w; }
                        }
                    }
                    tmem_store_32(trow + c * 32, sum);
                }
                tmem_store_wait();
            }
#pragma unroll 1
            for (int c = 0; c < TILE_COLS / 32; ++c) {
                const int col = c * 32, n = n0 + col;
                if (n >= p.N) break;
                float v[32];
                if (EPI == EPI_SWIGLU) {
                    float u[32];
                    tmem_load_32(trow + col, v);
                    tmem_load_32(trow + HALF + col, u);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        // gate and up are rounded to bfloat16 before the activation, as the
                        // unfused path stores them in between
                        const float gj = __bfloat162float(__float2bfloat16_rn(v[j]));
                        const float uj = __bfloat162float(__float2bfloat16_rn(u[j]));
                        // (approximate division: exact to 2 ulp of float, and without the slow path that
                        // the exact one takes when exp overflows the denominator; the quotient is 0 there)
                        v[j] = __fdividef(gj, 1.0f + expf(-gj)) * uj;
                    }
                } else {
                    tmem_load_32(trow + col, v);
                    tmem_load_wait();
                    if (p.bias) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (n + j < p.N) v[j] += __bfloat162float(p.bias[n + j]);
                    }
                }
                if (!p.tma_store) {
                    store_row_chunk(p, row0 + lane, n, v, vector_ok);
                    continue;
                }
                unsigned char* box = boxes + (groups & 1) * OUT_BOX_BYTES;
                const int half = c & 1;
                if (half == 0) {        // the store that read this box two groups ago has finished reading
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    __syncwarp();
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int j = q * 8;
                    uint4 w;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]), h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                    w.x = *reinterpret_cast<uint32_t*>(&h0); w.y = *reinterpret_cast<uint32_t*>(&h1);
                    w.z = *reinterpret_cast<uint32_t*>(&h2); w.w = *reinterpret_cast<uint32_t*>(&h3);
                    const int chunk = half * 4 + q;      // 16-byte chunk of the row, moved by the swizzle
                    *reinterpret_cast<uint4*>(box + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = w;
                }
                if (half == 1 || n + 32 >= p.N) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        // columns beyond N and rows beyond M are clipped by the copy engine
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                     ::"l"(&map_y), "r"(smem_addr(box)), "r"(n - half * 32), "r"(row0) : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    ++groups;
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_first_block(&acc_empty[buf]);
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();     // neither block frees tensor memory or leaves while the other may still signal it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// bf16 matrix [rows, cols] with `ld` elements between rows; boxes of 128 rows x 64 columns, 128-byte swizzle
static int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)ATOM_K, (cuuint32_t)HALF};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                               elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? 0 : ERR_BAD_ARGUMENT;
}

// bf16 output [rows, cols]: boxes of 32 rows x 64 columns, 128-byte swizzle, for the epilogue's stores
static int make_out_map(CUtensorMap* map, void* base, long long rows, long long cols, long long ld) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64, 32};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? 0 : ERR_BAD_ARGUMENT;
}

// Sets the kernel's shared-memory size once and asks how many pairs can run at the same time.
template <int EPI>
static int configure(int* max_pairs_out) {
    static int max_pairs = 0;
    if (max_pairs == 0) {
        auto kernel = gemm_tiles_kernel<EPI>;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        int device = 0, sms = 0, clusters = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(sms & ~1, 1, 1);
        config.blockDim = dim3(THREADS, 1, 1);
        config.dynamicSmemBytes = SMEM_BYTES;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        config.attrs = attr;
        config.numAttrs = 1;
        e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &config);
        if (e != cudaSuccess) return (int)e;
        if (clusters <= 0) return ERR_UNSUPPORTED;
        max_pairs = clusters;
    }
    *max_pairs_out = max_pairs;
    return 0;
}

// How the tiles after the last full round are shared out among `pairs` pairs: fills the sharing
// fields of p and returns the floats of workspace and the counters that the launch needs (0, 0
// when every tile is summed by one pair: no partial round, nothing to gain, or shares too short).
static void plan_sharing(TileGemmParams& p, long long tiles, int pairs, long long* floats, int* counters) {
    p.full_rounds = 0; p.shared_tiles = 0; p.share_pairs = 0; p.max_parts = 1;
    *floats = 0; *counters = 0;
    const int kblocks = (p.K + BK - 1) / BK;
    const int rest = (int)(tiles % pairs);
    // A partial round that occupies nine pairs in ten already gains too little for the workspace
    // traffic; and the adding of the parts hides under the whole tiles that follow, so without a
    // full round (fewer tiles than pairs: measured slower than leaving the tiles whole) nothing is shared.
    if (pairs < 2 || rest == 0 || tiles < pairs || rest * 10 >= pairs * 9) return;
    // What sharing saves is the idle share of a tile's time, and a tile's time goes with k (about
    // 20 us at k = 3,584); what it costs (the parts' trip through the workspace, about 10 us where
    // it is not hidden) does not: with short k it pays only when most pairs would idle (measured:
    // 112 tiles of k = 3,584 on 74 pairs gain nothing, 112 tiles of k = 18,944 gain 23 us of 203).
    if ((long long)(pairs - rest) * p.K < 1800LL * pairs) return;
    // at most four pairs per tile (the pair that arrives last adds their parts), shares of two k-blocks at least
    int share_pairs = pairs < 3 * rest ? pairs : 3 * rest;
    const long long units = (long long)rest * kblocks;
    if (share_pairs > units / 2) share_pairs = (int)(units / 2);
    int most = 1;
    for (;; --share_pairs) {
        if (share_pairs <= rest) return;
        most = 1;
        for (int r = 0; r < rest; ++r) {
            const int parts = share_of(units, share_pairs, (long long)(r + 1) * kblocks - 1) -
                              share_of(units, share_pairs, (long long)r * kblocks) + 1;
            if (parts > most) most = parts;
        }
        if (most <= 4) break;
    }
    p.full_rounds = (int)(tiles / pairs); p.shared_tiles = rest; p.share_pairs = share_pairs; p.max_parts = most;
    *floats = (long long)rest * most * 2 * HALF * TILE;
    *counters = rest * 2 * EPILOGUE_WARPS;
}

// Launch of `pairs` clusters of two blocks as a programmatic dependent of the kernel before it.
template <int EPI>
static int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const CUtensorMap& map_y, const TileGemmParams& p,
                  int pairs, cudaStream_t stream) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * pairs, 1, 1);
    config.blockDim = dim3(THREADS, 1, 1);
    config.dynamicSmemBytes = SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&config, gemm_tiles_kernel<EPI>, map_w, map_x, map_y, p);
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_gemm_tiles_map_bytes() { return (int)sizeof(CUtensorMap); }

// How many pairs of blocks run at the same time (also sets the kernels up, outside any stream
// capture); negative or a CUDA error code when the kernels cannot run here.
int fsie_gemm_tiles_pairs() {
    int plain = 0, swiglu = 0;
    int rc = configure<EPI_PLAIN>(&plain);
    if (rc == 0) rc = configure<EPI_SWIGLU>(&swiglu);
    if (rc != 0) return rc > 0 ? -rc : rc;
    return plain < swiglu ? plain : swiglu;
}

// Describe a bf16 weight matrix w[rows, K] (K contiguous) for the kernel below.
int fsie_gemm_tiles_weight_map(void* map_out, const void* w, long long rows, long long K) {
    if (K % 8 != 0 || (reinterpret_cast<uintptr_t>(w) & 15)) return ERR_BAD_ARGUMENT;
    CUtensorMap map;
    const int rc = make_map(&map, w, rows, K, K);
    if (rc == 0) memcpy(map_out, &map, sizeof(map));
    return rc;
}

// The pairs that a launch with these sizes uses, and what it needs to share out a partial last
// round of tiles: floats of workspace and ints of counters (both 0 when it does not share).
static int plan(int M, int N, int K, int swiglu, int blocks, TileGemmParams& p, int* pairs_out, long long* floats,
                int* counters) {
    int max_pairs = 0;
    const int rc = swiglu ? configure<EPI_SWIGLU>(&max_pairs) : configure<EPI_PLAIN>(&max_pairs);
    if (rc != 0) return rc;
    p.M = M; p.N = N; p.K = K;
    p.m_tiles = (M + TILE - 1) / TILE;
    p.n_tiles = swiglu ? (N + TILE / 2 - 1) / (TILE / 2) : (N + TILE - 1) / TILE;
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    int pairs = blocks / 2 > 0 ? blocks / 2 : 1;
    if (pairs > max_pairs) pairs = max_pairs;
    if (tiles < pairs) pairs = (int)tiles;
    *pairs_out = pairs;
    plan_sharing(p, tiles, pairs, floats, counters);
    return 0;
}

// What fsie_gemm_tiles needs beside its operands for these sizes: floats of workspace and ints of
// counters (zero before the first launch; every launch leaves them zero).  Both 0 where no tile is shared.
int fsie_gemm_tiles_workspace(int M, int N, int K, int swiglu, int blocks, long long* floats, int* counters) {
    *floats = 0; *counters = 0;
    if (M <= 0 || N <= 0 || K <= 0 || blocks <= 0) return 0;
    TileGemmParams p;
    int pairs = 0;
    return plan(M, N, K, swiglu, blocks, p, &pairs, floats, counters);
}

// y[M, N] = x[M, K] * w^T (+ bias), or for swiglu y[M, N] = silu(x w_gate^T) * (x w_up^T) with
// w = [gate rows (N); up rows (N)].  `blocks` is the size of the persistent grid (the number
// of SMs; it is cut to the pairs that can run at once and to the number of tiles).  workspace and
// counters: see fsie_gemm_tiles_workspace; with less than that (or null) every tile is summed by
// one pair, as if the last round were full.
int fsie_gemm_tiles(const void* weight_map, const void* x, long long ldx, void* y, long long ldy, const void* bias,
                    int M, int N, int K, int swiglu, int out_f32, int blocks, float* workspace,
                    long long workspace_floats, int* counters, int counters_len, int* error, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || blocks <= 0 || (swiglu && out_f32))
        return ERR_BAD_ARGUMENT;
    CUtensorMap map_w, map_x;
    memcpy(&map_w, weight_map, sizeof(map_w));
    int rc = make_map(&map_x, x, M, K, ldx);
    if (rc != 0) return rc;
    TileGemmParams p;
    int pairs = 0, need_counters = 0;
    long long need_floats = 0;
    rc = plan(M, N, K, swiglu, blocks, p, &pairs, &need_floats, &need_counters);
    if (rc != 0) return rc;
    if (p.share_pairs > 0 && (!workspace || !counters || workspace_floats < need_floats || counters_len < need_counters))
        p.share_pairs = 0;
    p.workspace = workspace; p.counters = counters;
    p.y = y; p.ldy = ldy; p.bias = (const bf16*)bias;
    p.up_row0 = N; p.out_f32 = out_f32; p.error = error;
    // the copy engine writes y when its rows start on 16-byte boundaries; else the lanes store their rows
    p.tma_store = !out_f32 && ldy % 8 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
    CUtensorMap map_y = map_x;
    if (p.tma_store) {
        rc = make_out_map(&map_y, y, M, N, ldy);
        if (rc != 0) return rc;
    }
    return swiglu ? launch<EPI_SWIGLU>(map_w, map_x, map_y, p, pairs, stream) : launch<EPI_PLAIN>(map_w, map_x, map_y, p, pairs, stream);
}

}  // extern "C"
