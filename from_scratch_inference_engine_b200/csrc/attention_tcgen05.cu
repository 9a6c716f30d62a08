// Causal grouped-query attention for prompt portions on the 5th-generation tensor cores:
// scores and outputs are accumulated in tensor memory by tcgen05.mma, keys and values arrive
// by TMA, bfloat16 storage, 32-bit scores / softmax statistics / accumulation.
// Compiled per head size (-DHEAD_DIM=64 or 128).
//
// A block owns 256 query rows of one request and one kv head - a row is a (new token, head of
// the group) pair as in attention_mma.cu - as two streams A and B of 128 rows each (one
// tensor-memory lane per row), and walks the keys in tiles of 128.  Both streams use the same
// key and value tiles, so each tile is fetched once for 256 rows, and while the softmax of one
// stream runs on the CUDA cores the tensor core works for the other:
//
//   producer warp   TMA: one cp.async.bulk.tensor per page and 128-byte column half; K and V
//                   tiles take turns in a ring of five slots (full/empty mbarriers), 128-byte swizzle
//   MMA warp        S_X = Q_X K_i^T  (128 x 128 x head_dim, A and B K-major from shared memory) into
//                   the stream's score columns of tensor memory; O_X += P_X V_i  (128 x head_dim x
//                   128, A = P from tensor memory, B = V MN-major straight from its [key][dim]
//                   tile); for each stream in turn: P V of tile i, then Q K^T of tile i + 1.
//                   (A second issuing thread, one per stream, measured slower: 685 against 833
//                   TFLOP/s at 8,192 tokens.)
//   2 x 4 softmax   one thread per row: read S, mask, running maximum and sum, write P as bfloat16
//   warps           pairs over the first half of the S columns it has just read (shared memory is
//                   the scarce resource here: operands read by the MMAs, tiles written by TMA;
//                   P never passes through it), rescale O in tensor memory when a row's maximum
//                   moved, finally normalise O and store it (or a partial result when the key
//                   range is split)
//
// Formula: src/model/nn.cpp:151-226 of the reference, as a running softmax.
// Every wait on an mbarrier is bounded; when one runs out *error is set, all roles leave their
// loops, tensor memory is freed and the kernel returns.
#include "common.cuh"
#include "attention_params.cuh"
#include "tma.cuh"
#include <math.h>
#include <string.h>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "head size 64 or 128");

namespace fsie {

constexpr int HD = HEAD_DIM;
constexpr int BM = 128;                 // query rows per stream = tensor-memory lanes
constexpr int STREAMS = 2;              // streams of query rows per block
constexpr int BN = 128;                 // keys per tile
constexpr int SLOTS = 5;                // ring of key / value tiles: K_i, V_i, K_i+1, ...
constexpr int SOFTMAX_WARPS = 4 * STREAMS;
constexpr int THREADS = 64 + 32 * SOFTMAX_WARPS;
constexpr int HALVES = HD / 64;         // 128-byte column halves of a row of head_dim elements
constexpr int ATOM_BYTES = 128 * 128;   // 128 rows x 128 bytes: one swizzled block
constexpr int Q_BYTES = HALVES * ATOM_BYTES;           // one stream's queries
constexpr int KV_BYTES = HALVES * ATOM_BYTES;          // one K or V tile
constexpr int TILE_BYTES = STREAMS * Q_BYTES + SLOTS * KV_BYTES;
// Barriers come first in the block's (dynamic only) shared memory, the swizzled tiles follow at
// the next 1,024-byte boundary.  With head size 128 this is all the shared memory an SM offers
// to a block (227 KB), so the kernel has no static shared memory and relies on the window
// starting on such a boundary; it checks and refuses otherwise.
struct Control {
    uint64_t ring_full[SLOTS], ring_empty[SLOTS], s_full[STREAMS], p_ready[STREAMS], o_done[STREAMS], q_ready;
    uint32_t tmem_slot;
    int abort_flag;
};
static_assert(sizeof(Control) <= 1024, "control block");
constexpr int SMEM_BYTES = 1024 + TILE_BYTES;
constexpr uint32_t TMEM_COLS = 512;     // S_A | S_B | O_A | O_B, 128 columns each; P_X (bfloat16 pairs) over the first 64 of S_X
constexpr uint32_t COL_S = 0, COL_O = STREAMS * BN;
enum { ERR_TC_PRODUCER = 31, ERR_TC_MMA = 32, ERR_TC_SOFTMAX = 33, ERR_TC_LAYOUT = 34 };

struct TcExtra { int entries, entry; int* error; };
#define TC_MARK(slot) do { } while (0)

}  // namespace fsie
#include "attention_combine.cuh"
namespace fsie {

// 64-bit shared-memory matrix descriptors (version 1, 128-byte swizzle).
// K-major: rows of 128 bytes, 8-row groups 1,024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(const void* p) {
    return (uint64_t)((smem_addr(p) & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major (the tile is stored [k][mn] with 64 mn-elements = 128 bytes per k): 8 k-rows are a
// 1,024-byte block (stride byte offset), the next 64 mn-elements are a whole block column
// further (leading byte offset).
__device__ __forceinline__ uint64_t desc_mn_major(const void* p, uint32_t mn_block_bytes) {
    return (uint64_t)((smem_addr(p) & 0x3FFFF) >> 4) | ((uint64_t)(mn_block_bytes >> 4) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// instruction descriptor: D float, A and B bfloat16, M x N; b_mn_major selects an MN-major B
__device__ __forceinline__ uint32_t idesc_bf16(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// the same with A[128, 16] read from tensor memory (lane = row, 8 columns of bfloat16 pairs)
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// issue a read of 32 columns; the registers are valid only after tmem_wait_ld()
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32_issue(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
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
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float fast_exp2(float v) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
// byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a 128-byte-swizzled block
__device__ __forceinline__ int swizzled(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

__global__ void __launch_bounds__(THREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap pages_map, const AttnParams p, const TcExtra x) {
    extern __shared__ __align__(1024) unsigned char smem_all[];
    Control& ctl = *reinterpret_cast<Control*>(smem_all);
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_all) + sizeof(Control) + 1023) & ~uintptr_t(1023));
    if (smem + TILE_BYTES > smem_all + SMEM_BYTES) {        // the window does not start on a 1,024-byte boundary
        if (threadIdx.x == 0) atomicExch(x.error, ERR_TC_LAYOUT);
        return;
    }
    unsigned char* q_s = smem;                               // [stream][HALVES][128 rows][128 B]
    unsigned char* ring = q_s + STREAMS * Q_BYTES;           // [slot][HALVES][128 keys][128 B]
    int& abort_flag = ctl.abort_flag;

    // Blocks are handed out in the order of blockIdx.x, and the caller lists the tiles with the most
    // keys first: all kv heads of the longest tile start first, so that the last wave is short.
    const int tile = blockIdx.x / p.kv_heads, kvh = blockIdx.x % p.kv_heads, split = blockIdx.z;
    const int group = p.heads / p.kv_heads;
    const int item = p.tile_item[tile];
    const int row0 = p.tile_row0[tile];
    const int qstart = p.item_qstart[item], qlen = p.item_qlen[item], pos0 = p.item_pos0[item];
    const int nrows = min(STREAMS * BM, qlen * group - row0);
    const int streams = nrows > BM ? 2 : 1;                  // a short tile leaves stream B idle
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bf16* q = (const bf16*)p.q;
    const int* bt = p.block_tables + (size_t)item * p.bt_stride;

    const int pos_first = pos0 + row0 / group;
    const int pos_last = pos0 + (row0 + nrows - 1) / group;
    int kbegin = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    // tiles hold whole pages, and keys before the window are masked: the range starts on a tile
    // boundary before it is split, so that the splits' ranges stay disjoint
    kbegin = kbegin / BN * BN;
    int kend = pos_last + 1;
    if (p.nsplit > 1) {
        const int span = kend - kbegin;
        int chunk = (span + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + BN - 1) / BN) * BN;
        const int b = kbegin + split * chunk;
        kend = min(kend, b + chunk);
        kbegin = b;
    }
    const int ntiles = kend > kbegin ? (kend - kbegin + BN - 1) / BN : 0;

    // ---- set-up: barriers and tensor memory; then the producer starts fetching keys at once while
    // the other warps bring the query rows into the swizzled K-major layout
    if (tid == 0) {
        for (int s = 0; s < SLOTS; ++s) { mbar_init(&ctl.ring_full[s], 1); mbar_init(&ctl.ring_empty[s], 1); }
        for (int st = 0; st < STREAMS; ++st) {
            mbar_init(&ctl.s_full[st], 1); mbar_init(&ctl.p_ready[st], BM); mbar_init(&ctl.o_done[st], 1);
        }
        mbar_init(&ctl.q_ready, THREADS - 32);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&ctl.tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctl.tmem_slot;
    if (warp != 0) {
        // all of a thread's loads go out before the first of its stores: one trip to memory, not one
        // per 16 bytes
        constexpr int CHUNKS = STREAMS * BM * (HD / 8), LOADERS = THREADS - 32;
        constexpr int PER_THREAD = (CHUNKS + LOADERS - 1) / LOADERS;
        uint4 held[PER_THREAD];
#pragma unroll
        for (int j = 0; j < PER_THREAD; ++j) {
            const int e = tid - 32 + j * LOADERS;
            const int r = e / (HD / 8), c = e - r * (HD / 8);     // 16-byte chunk c of row r of the block
            held[j] = make_uint4(0, 0, 0, 0);
            if (e < CHUNKS && r < nrows) {
                const int row = row0 + r;
                const int tok = qstart + row / group, h = kvh * group + row % group;
                held[j] = *reinterpret_cast<const uint4*>(q + (size_t)tok * p.q_ld + h * HD + c * 8);
            }
        }
#pragma unroll
        for (int j = 0; j < PER_THREAD; ++j) {
            const int e = tid - 32 + j * LOADERS;
            const int r = e / (HD / 8), c = e - r * (HD / 8);
            if (e < CHUNKS)
                *reinterpret_cast<uint4*>(q_s + (r / BM) * Q_BYTES + (c >> 3) * ATOM_BYTES + swizzled(r % BM, c & 7)) = held[j];
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic writes before async-proxy reads
        mbar_arrive(&ctl.q_ready);
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        // ring entry 2 i is K of tile i, entry 2 i + 1 its V.  Lane j looks up and fetches page j of
        // the tile: the table reads and the copy instructions go out side by side.
        const int ps = p.page_size, pages_per_tile = BN / ps;
        const long long rows_per_page = (long long)x.entries * 2 * p.kv_heads * ps;
        const long long k_row0 = ((long long)x.entry * 2) * p.kv_heads * ps + (long long)kvh * ps;
        const long long v_row0 = k_row0 + (long long)p.kv_heads * ps;
        for (int i = 0; i < ntiles; ++i) {
            // Every part of a tile is fetched, so that what the MMAs read is always finite: where the
            // tile reaches beyond the last key, or into pages that a window has given back, the page
            // of the last key stands in (those keys are masked).
            const int key = kbegin + i * BN + lane * ps;
            int page = -1;
            if (lane < pages_per_tile) {                  // before the wait: overlaps it
                page = key < kend ? bt[key / ps] : -1;
                if (page < 0) page = bt[(kend - 1) / ps];
            }
            const int wanted = __popc(__ballot_sync(0xffffffffu, page >= 0));
            bool ok = true;
#pragma unroll
            for (int kv = 0; kv < 2 && ok; ++kv) {
                const int e = 2 * i + kv, s = e % SLOTS;
                if (lane == 0 && e >= SLOTS) ok = mbar_wait(&ctl.ring_empty[s], ((e / SLOTS) - 1) & 1);
                ok = __shfl_sync(0xffffffffu, ok, 0) && !*(volatile int*)&abort_flag;
                if (!ok) break;
                if (lane == 0) mbar_expect_tx(&ctl.ring_full[s], (uint32_t)wanted * ps * HD * 2);
                __syncwarp();
                if (page >= 0) {
                    unsigned char* dst = ring + (size_t)s * KV_BYTES + lane * ps * 128;
                    const long long row = (long long)page * rows_per_page + (kv ? v_row0 : k_row0);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h) tma_load_2d(dst + h * ATOM_BYTES, &pages_map, h * 64, (int)row, &ctl.ring_full[s]);
                }
            }
            if (!ok) {
                if (lane == 0) { atomicExch(x.error, ERR_TC_PRODUCER); atomicExch(&abort_flag, 1); }
                break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && ntiles > 0) {
            const uint32_t idesc_s = idesc_bf16(BM, BN, 0), idesc_o = idesc_bf16(BM, HD, 1);
            bool ok = true;
            auto ring_wait = [&](int e) {            // the tile of ring entry e has arrived
                if (!mbar_wait(&ctl.ring_full[e % SLOTS], (e / SLOTS) & 1)) {
                    atomicExch(x.error, ERR_TC_MMA); atomicExch(&abort_flag, 1); ok = false;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            };
            // Descriptors differ from one MMA to the next only by a constant in their address field
            // (16-byte units): the issuing thread adds it to a base made once.
            const uint64_t q_base = desc_k_major(q_s), k_base = desc_k_major(ring), v_base = desc_mn_major(ring, ATOM_BYTES);
            auto scores = [&](int st, int i) {       // S_st = Q_st K_i^T
                const uint64_t qd = q_base + (uint64_t)(st * (Q_BYTES >> 4));
                const uint64_t kd = k_base + (uint64_t)(((2 * i) % SLOTS) * (KV_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    // 16 elements along the head: 32 bytes inside the swizzled row; 64: the next block
                    const uint32_t step = (k >> 2) * (ATOM_BYTES >> 4) + 2 * (k & 3);
                    mma_ss(tmem + COL_S + st * BN, qd + step, kd + step, idesc_s, k > 0);
                }
                mma_commit(&ctl.s_full[st]);
                if (st == streams - 1) mma_commit(&ctl.ring_empty[(2 * i) % SLOTS]);     // K_i may be overwritten
            };
            if (!mbar_wait(&ctl.q_ready, 0)) {
                atomicExch(x.error, ERR_TC_MMA); atomicExch(&abort_flag, 1); ok = false;
            }
            ring_wait(0);
            for (int st = 0; st < streams && ok; ++st) scores(st, 0);
            for (int i = 0; i < ntiles && ok; ++i) {
                for (int st = 0; st < streams && ok; ++st) {
                    if (!mbar_wait(&ctl.p_ready[st], i & 1)) {
                        atomicExch(x.error, ERR_TC_MMA); atomicExch(&abort_flag, 1); ok = false; break;
                    }
                    if (st == 0) ring_wait(2 * i + 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t vd = v_base + (uint64_t)(((2 * i + 1) % SLOTS) * (KV_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < BN / 16; ++k) {         // 16 keys per instruction
                        // 16 keys of P: 8 columns of bfloat16 pairs in the stream's score columns;
                        // 16 keys of V: 16 rows of 128 bytes
                        mma_ts(tmem + COL_O + st * BN, tmem + COL_S + st * BN + k * 8, vd + (uint64_t)(k * (16 * 128 >> 4)),
                               idesc_o, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    if (i + 1 == ntiles) mma_commit(&ctl.o_done[st]);       // O_st is complete
                    if (st == streams - 1) mma_commit(&ctl.ring_empty[(2 * i + 1) % SLOTS]);    // V_i may be overwritten
                    if (i + 1 < ntiles) {                       // the stream's next scores, while the other's softmax runs
                        if (st == 0) ring_wait(2 * i + 2);
                        if (!ok) break;
                        scores(st, i + 1);
                    }
                }
            }
        }
    } else if ((warp - 2) / 4 < streams) {
        // ------------------------------------------------------------------ softmax, one thread per row
        const int st = (warp - 2) / 4;                      // stream A or B
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                  // row of the stream = tensor-memory lane
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        const uint32_t s_addr = lane_base + COL_S + st * BN, o_addr = lane_base + COL_O + st * BN;
        const bool valid = st * BM + r < nrows;
        const int pos = valid ? pos0 + (row0 + st * BM + r) / group : -1;
        const int lowest = p.window > 0 ? pos - p.window : -1;       // keys <= this are unseen
        const float sc = p.scale * 1.4426950408889634f;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int i = 0; i < ntiles && ok; ++i) {
            // (decisions to give up are taken by whole warps: the tensor-memory accesses below are
            // warp-collective)
            if (!__all_sync(0xffffffffu, mbar_wait(&ctl.s_full[st], i & 1))) {
                if (lane == 0) atomicExch(x.error, ERR_TC_SOFTMAX);
                atomicExch(&abort_flag, 1); ok = false; break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            TC_MARK(0);
            const int k0 = kbegin + i * BN;
            // the row's 128 scores in registers: four reads in flight, one wait
            uint32_t sr[BN];
#pragma unroll
            for (int c = 0; c < BN; c += 32) tmem_ld32_issue(s_addr + c, sr + c);
            tmem_wait_ld();
            TC_MARK(1);
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains, not one
            const bool clear = k0 + BN - 1 < kend && k0 + BN - 1 <= pos && k0 > lowest;   // nothing to mask
            if (__all_sync(0xffffffffu, clear || !valid)) {
#pragma unroll
                for (int j = 0; j < BN; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(sr[j]));
            } else {
#pragma unroll
                for (int j = 0; j < BN; ++j) {
                    const int key = k0 + j;
                    const bool seen = key < kend && key <= pos && key > lowest;
                    if (!seen) sr[j] = 0xff800000u;                    // -inf
                    mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(sr[j]));
                }
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            if (!valid) mx = -INFINITY;
            // The reference point of the exponentials moves only when the row's maximum has grown
            // by more than 2^8 since it was set: until then p may exceed 1 (by at most 256x, exact
            // enough in float and bfloat16), and O and the row sum need no rescaling.
            float m_new = m_run;
            if (mx > m_run && (m_run == -INFINITY || (mx - m_run) * sc > 8.f)) m_new = mx;
            const float base = m_new == -INFINITY ? 0.f : m_new * sc;
            const float corr = m_new == m_run ? 1.f : fast_exp2(m_run * sc - base);    // m_run = -inf gives 0
            const bool rescale = i > 0 && __any_sync(0xffffffffu, valid && corr != 1.f);
            TC_MARK(2);
            // O and P of this stream were last touched by the P V of tile i - 1, which the tensor core
            // finished before it wrote this S: neither needs a wait of its own.
            TC_MARK(3);
            if (rescale) {
#pragma unroll 1
                for (int c = 0; c < HD; c += 32) {
                    uint32_t orr[32];
                    tmem_ld32_issue(o_addr + c, orr);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) orr[j] = __float_as_uint(__uint_as_float(orr[j]) * corr);
                    tmem_st32_issue(o_addr + c, orr);
                    tmem_wait_st();
                }
            }
            // p = exp2(s * sc - base), row sum, P as bfloat16 pairs (key 2 c low, key 2 c + 1 high in
            // column c) over the registers that held the scores
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < BN; j += 2) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(sr[j]), sc, -base));
                const float p1 = fast_exp2(fmaf(__uint_as_float(sr[j + 1]), sc, -base));
                sum4[(j >> 1) & 1] += p0;
                sum4[2 + ((j >> 1) & 1)] += p1;
                __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                sr[j >> 1] = *reinterpret_cast<uint32_t*>(&h2);
            }
#pragma unroll
            for (int c = 0; c < BN / 2; c += 32) tmem_st32_issue(s_addr + c, sr + c);
            tmem_wait_st();
            const float sum = valid ? (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]) : 0.f;
            l_run = l_run * corr + sum;
            m_run = m_new;
            TC_MARK(4);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");  // P (and a rescaled O) before the next MMA
            mbar_arrive(&ctl.p_ready[st]);
            TC_MARK(5);
        }
        // ---- the last P V, then normalise and store (or hand a partial result to the merge)
        bool have = ok && ntiles > 0;
        if (have && !__all_sync(0xffffffffu, mbar_wait(&ctl.o_done[st], 0))) {
            if (lane == 0) atomicExch(x.error, ERR_TC_SOFTMAX);
            atomicExch(&abort_flag, 1); have = false;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int row = row0 + (valid ? st * BM + r : 0);
        const int tok = qstart + row / group, h = kvh * group + row % group;
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
            float v[32];
            if (have) tmem_ld32(o_addr + c, v);       // warp-collective: every lane takes part
            else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.f;
            }
            if (!valid) continue;
            if (p.nsplit == 1) {
                bf16* dst = (bf16*)p.out + (size_t)tok * p.out_ld + h * HD + c;
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {
                    uint4 packed;
                    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        h2[j] = __floats2bfloat162_rn(v[g8 * 8 + 2 * j] * inv, v[g8 * 8 + 2 * j + 1] * inv);
                    *reinterpret_cast<uint4*>(dst + g8 * 8) = packed;
                }
            } else {
                const size_t idx = ((size_t)split * p.tokens + tok) * p.heads + h;
                float* dst = p.part_o + idx * HD + c;
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
        }
        if (valid && p.nsplit > 1) {
            const size_t idx = ((size_t)split * p.tokens + tok) * p.heads + h;
            p.part_ml[idx * 2] = m_run == -INFINITY ? -INFINITY : m_run * p.scale;
            p.part_ml[idx * 2 + 1] = l_run;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}


// =====================================================================================
// Decoded tokens (and portions of up to 16 rows): the keys are the M side.
//
// A decoded token has as many query rows as its group has heads (5-8), far too few for the
// 128 rows of an MMA, and with mma.sync tiles the CUDA cores spend more instructions per key
// than the memory system needs time to deliver it.  Here a tile is 128 keys x 16 rows:
//
//   S^T[key, row] = K_tile[128 keys, head] . Q^T         (A = the K tile, K-major, as TMA wrote it;
//                                                         B = 16 query rows, K-major; N = 16)
//   O^T[dim, row] += V_tile^T[128 dims, 128 keys] . P^T  (A = the V tile as it lies, [key][dim] =
//                                                         MN-major; B = P^T [row][key], K-major)
//
// so every byte of K and V is read from shared memory once by the tensor core, and the 128
// softmax threads hold one key each: 16 scores per thread and tile.  The maximum of a row over
// the keys of a tile is found with a warp reduction and a shared atomic per row; the row sums
// stay per thread until the end.  As in the kernel above the reference point of a row's
// exponentials moves only when its maximum has grown by more than 2^8.
//
//   producer warp   TMA, K and V tiles take turns in a ring of DSLOTS slots
//   MMA warp        scores of tile i + 1 (second S buffer) are issued before P V of tile i
//   4 softmax warps thread t = key t of the tile = tensor-memory lane t; at the end lane t holds
//                   dimension t of the 16 outputs
#if HEAD_DIM == 128
namespace dec {

constexpr int KEYS = 128;               // keys per tile
constexpr int ROWS = 16;                // query rows per tile
constexpr int DSLOTS = 3;               // ring of K / V tiles; with 3 two blocks fit on an SM
constexpr int DTHREADS = 64 + 128;
constexpr int QP_ATOM = ROWS * 128;     // 16 rows x 128 bytes of a K-major operand with N = 16
constexpr int DQ_BYTES = HALVES * QP_ATOM;
constexpr int DP_BYTES = (KEYS / 64) * QP_ATOM;
constexpr int DTILE_BYTES = DQ_BYTES + DP_BYTES + DSLOTS * KV_BYTES;
struct DControl {
    uint64_t ring_full[DSLOTS], ring_empty[DSLOTS], s_full[2], p_ready, pv_done, q_ready;
    uint32_t tmem_slot;
    int abort_flag;
    int row_max[1][ROWS];               // a tile's row maxima (as ordered integers), when reference points move
    float row_sum[4][ROWS];             // the softmax warps' sums at the end
};
static_assert(sizeof(DControl) <= 1024, "control block");
constexpr int DSMEM_BYTES = 1024 + DTILE_BYTES;
constexpr uint32_t DTMEM_COLS = 64;     // S (tile parity 0) | S (parity 1) | O, 16 columns each
constexpr uint32_t DCOL_O = 32;
enum { ERR_TCD_PRODUCER = 35, ERR_TCD_MMA = 36, ERR_TCD_SOFTMAX = 37, ERR_TCD_LAYOUT = 38 };

// floats as integers of the same order (for atomicMax / redux)
__device__ __forceinline__ int ordered(float f) { const int i = __float_as_int(f); return i >= 0 ? i : i ^ 0x7fffffff; }
__device__ __forceinline__ float unordered(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff); }

__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16_issue(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
// all 128 softmax threads meet; returns whether any of them brought `flag`
__device__ __forceinline__ bool softmax_meet(bool flag) {
    uint32_t any;
    asm volatile("{\n .reg .pred pin, pout;\n setp.ne.u32 pin, %1, 0;\n bar.red.or.pred pout, 1, 128, pin;\n selp.u32 %0, 1, 0, pout;\n}\n"
                 : "=r"(any) : "r"((uint32_t)flag) : "memory");
    return any != 0;
}

__global__ void __launch_bounds__(DTHREADS, DSLOTS <= 3 ? 2 : 1)
attn_tc_decode_kernel(const __grid_constant__ CUtensorMap pages_map, const AttnParams p, const TcExtra x) {
    extern __shared__ __align__(1024) unsigned char smem_all[];
    DControl& ctl = *reinterpret_cast<DControl*>(smem_all);
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_all) + sizeof(DControl) + 1023) & ~uintptr_t(1023));
    if (smem + DTILE_BYTES > smem_all + DSMEM_BYTES) {       // the window does not start on a 1,024-byte boundary
        if (threadIdx.x == 0) atomicExch(x.error, ERR_TCD_LAYOUT);
        return;
    }
    unsigned char* q_s = smem;                               // [HALVES][16 rows][128 B]
    unsigned char* p_s = q_s + DQ_BYTES;                     // [2 halves of the keys][16 rows][128 B]
    unsigned char* ring = p_s + DP_BYTES;                    // [slot][HALVES][128 keys][128 B]
    int& abort_flag = ctl.abort_flag;

    const int kvh = blockIdx.x, tile = blockIdx.y, split = blockIdx.z;
    const int group = p.heads / p.kv_heads;
    const int item = p.tile_item[tile];
    const int row0 = p.tile_row0[tile];
    const int qstart = p.item_qstart[item], qlen = p.item_qlen[item], pos0 = p.item_pos0[item];
    const int nrows = min(ROWS, qlen * group - row0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bf16* q = (const bf16*)p.q;
    const int* bt = p.block_tables + (size_t)item * p.bt_stride;

    const int pos_first = pos0 + row0 / group;
    const int pos_last = pos0 + (row0 + nrows - 1) / group;
    int kbegin = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    // tiles hold whole pages, and keys before the window are masked: the range starts on a tile
    // boundary before it is split, so that the splits' ranges stay disjoint
    kbegin = kbegin / KEYS * KEYS;
    int kend = pos_last + 1;
    if (p.nsplit > 1) {
        const int span = kend - kbegin;
        int chunk = (span + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + KEYS - 1) / KEYS) * KEYS;
        const int b = kbegin + split * chunk;
        kend = min(kend, b + chunk);
        kbegin = b;
    }
    const int ntiles = kend > kbegin ? (kend - kbegin + KEYS - 1) / KEYS : 0;

    if (tid == 0) {
        for (int s = 0; s < DSLOTS; ++s) { mbar_init(&ctl.ring_full[s], 1); mbar_init(&ctl.ring_empty[s], 1); }
        mbar_init(&ctl.s_full[0], 1); mbar_init(&ctl.s_full[1], 1);
        mbar_init(&ctl.p_ready, 128); mbar_init(&ctl.pv_done, 1); mbar_init(&ctl.q_ready, 128);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid == 32) asm volatile("prefetch.tensormap [%0];" ::"l"(&pages_map) : "memory");
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&ctl.tmem_slot)), "r"(DTMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctl.tmem_slot;
    grid_dependents_go();
    // Under programmatic dependent launch the kernel before this one, which writes this step's
    // queries, keys and values, may still be running.  The lists and block tables were staged
    // before the step, and keys older than every new token of the request were written by earlier
    // steps: the producer fetches tiles of only such keys at once and waits before the first tile
    // with new ones; everyone else waits here.
    if (warp != 0) grid_dependency_wait();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        // ring entry 2 i is K of tile i, entry 2 i + 1 its V; lane j fetches page j of the tile
        const int ps = p.page_size, pages_per_tile = KEYS / ps;
        const long long rows_per_page = (long long)x.entries * 2 * p.kv_heads * ps;
        const long long k_row0 = ((long long)x.entry * 2) * p.kv_heads * ps + (long long)kvh * ps;
        const long long v_row0 = k_row0 + (long long)p.kv_heads * ps;
        bool waited = false;
        // every part of a tile is fetched (finite operands): beyond the last key, or where a window
        // has given pages back, the page of the last key stands in; those keys are masked.  The
        // table entries of a tile are read one tile ahead of their use.
        const int last_page = ntiles > 0 ? bt[(kend - 1) / ps] : -1;
        auto look_up = [&](int i) {
            const int key = kbegin + i * KEYS + lane * ps;
            return (lane < pages_per_tile && i < ntiles && key < kend) ? bt[key / ps] : -1;
        };
        int page_ahead = look_up(0);
        for (int i = 0; i < ntiles; ++i) {
            if (!waited && kbegin + (i + 1) * KEYS > pos0) { grid_dependency_wait(); waited = true; }
            int page = page_ahead;
            page_ahead = look_up(i + 1);
            if (lane < pages_per_tile && page < 0) page = last_page;
            const int wanted = __popc(__ballot_sync(0xffffffffu, page >= 0));
            bool ok = true;
#pragma unroll
            for (int kv = 0; kv < 2 && ok; ++kv) {
                const int e = 2 * i + kv, s = e % DSLOTS;
                if (lane == 0 && e >= DSLOTS) ok = mbar_wait(&ctl.ring_empty[s], ((e / DSLOTS) - 1) & 1);
                ok = __shfl_sync(0xffffffffu, ok, 0) && !*(volatile int*)&abort_flag;
                if (!ok) break;
                if (lane == 0) mbar_expect_tx(&ctl.ring_full[s], (uint32_t)wanted * ps * HD * 2);
                __syncwarp();
                if (page >= 0) {
                    unsigned char* dst = ring + (size_t)s * KV_BYTES + lane * ps * 128;
                    const long long row = (long long)page * rows_per_page + (kv ? v_row0 : k_row0);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h) tma_load_2d(dst + h * ATOM_BYTES, &pages_map, h * 64, (int)row, &ctl.ring_full[s]);
                }
            }
            if (!ok) {
                if (lane == 0) { atomicExch(x.error, ERR_TCD_PRODUCER); atomicExch(&abort_flag, 1); }
                break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && ntiles > 0) {
            const uint32_t idesc_s = idesc_bf16(KEYS, ROWS, 0);                  // A = K tile, B = Q: both K-major
            const uint32_t idesc_o = idesc_bf16(HD, ROWS, 0) | (1u << 15);       // A = V tile, MN-major
            bool ok = true;
            auto give_up = [&]() { atomicExch(x.error, ERR_TCD_MMA); atomicExch(&abort_flag, 1); ok = false; };
            auto ring_wait = [&](int e) {
                if (!mbar_wait(&ctl.ring_full[e % DSLOTS], (e / DSLOTS) & 1)) give_up();
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            };
            const uint64_t q_base = desc_k_major(q_s), p_base = desc_k_major(p_s);
            const uint64_t k_base = desc_k_major(ring), v_base = desc_mn_major(ring, ATOM_BYTES);
            auto scores = [&](int i) {               // S^T (parity of i) = K_i Q^T
                const uint64_t kd = k_base + (uint64_t)(((2 * i) % DSLOTS) * (KV_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)    // 16 elements along the head per instruction
                    mma_ss(tmem + (i & 1) * ROWS, kd + (uint64_t)((k >> 2) * (ATOM_BYTES >> 4) + 2 * (k & 3)),
                           q_base + (uint64_t)((k >> 2) * (QP_ATOM >> 4) + 2 * (k & 3)), idesc_s, k > 0);
                mma_commit(&ctl.s_full[i & 1]);
                mma_commit(&ctl.ring_empty[(2 * i) % DSLOTS]);                   // K_i may be overwritten
            };
            if (!mbar_wait(&ctl.q_ready, 0)) give_up();
            if (ok) ring_wait(0);
            if (ok) scores(0);
            for (int i = 0; i < ntiles && ok; ++i) {
                if (i + 1 < ntiles) {                // the next scores, while the softmax works on these
                    ring_wait(2 * i + 2);
                    if (!ok) break;
                    scores(i + 1);
                }
                if (!mbar_wait(&ctl.p_ready, i & 1)) { give_up(); break; }
                ring_wait(2 * i + 1);
                if (!ok) break;
                const uint64_t vd = v_base + (uint64_t)(((2 * i + 1) % DSLOTS) * (KV_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < KEYS / 16; ++k)  // 16 keys per instruction: 16 rows of 128 bytes of V
                    mma_ss(tmem + DCOL_O, vd + (uint64_t)(k * (16 * 128 >> 4)),
                           p_base + (uint64_t)((k >> 2) * (QP_ATOM >> 4) + 2 * (k & 3)), idesc_o, (i > 0 || k > 0) ? 1u : 0u);
                mma_commit(&ctl.pv_done);
                mma_commit(&ctl.ring_empty[(2 * i + 1) % DSLOTS]);               // V_i may be overwritten
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax: one key per thread
        const int quarter = warp & 3;
        const int t = quarter * 32 + lane;                  // key of the tile = tensor-memory lane
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        // the query rows, K-major and swizzled (rows beyond the tile's count are zero)
#pragma unroll
        for (int j = 0; j < ROWS * (HD / 8) / 128; ++j) {
            const int e = t + j * 128;
            const int r = e / (HD / 8), c = e - r * (HD / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < nrows) {
                const int row = row0 + r;
                const int tok = qstart + row / group, h = kvh * group + row % group;
                v = *reinterpret_cast<const uint4*>(q + (size_t)tok * p.q_ld + h * HD + c * 8);
            }
            *reinterpret_cast<uint4*>(q_s + (c >> 3) * QP_ATOM + swizzled(r, c & 7)) = v;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(&ctl.q_ready);

        int pos[ROWS], low[ROWS];
        int pos_min = 0x7fffffff, low_max = -1;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            pos[r] = r < nrows ? pos0 + (row0 + r) / group : -1;
            low[r] = p.window > 0 ? pos[r] - p.window : -1;      // keys <= this are unseen
            if (r < nrows) { pos_min = min(pos_min, pos[r]); low_max = max(low_max, low[r]); }
        }
        const float sc = p.scale * 1.4426950408889634f;
        // base[r]: the reference point of row r's exponentials in base-2 units (-inf: none yet)
        float base[ROWS], l_run[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) { base[r] = -INFINITY; l_run[r] = 0.f; }
        // where P^T [row][key] takes this thread's key: 2 bytes in each row's 128-byte line
        unsigned char* p_mine = p_s + (t >> 6) * QP_ATOM + (t & 7) * 2;
        const int p_chunk = (t & 63) >> 3;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)          // rows beyond the tile's count stay zero
            if (r >= nrows) *reinterpret_cast<bf16*>(p_mine + r * 128 + ((p_chunk ^ (r & 7)) << 4)) = __float2bfloat16_rn(0.f);
        bool fail = false, left = false;
        for (int i = 0; i < ntiles; ++i) {
            if (!mbar_wait(&ctl.s_full[i & 1], (i >> 1) & 1)) fail = true;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            TC_MARK(0);
            uint32_t sr[ROWS];
            tmem_ld16_issue(lane_base + (i & 1) * ROWS, sr);
            tmem_wait_ld();
            TC_MARK(1);
            const int k0 = kbegin + i * KEYS, key = k0 + t;
            const bool clear = k0 + KEYS - 1 < kend && k0 + KEYS - 1 <= pos_min && k0 > low_max;   // nothing to mask
            // Exponent of every score against its row's reference point.  The point moves only when
            // some score lies more than 2^8 above it (or the row has none yet): p may exceed 1 by
            // at most 256x, exact enough in float and bfloat16, and in almost every tile nobody
            // needs the row maxima, O and the row sums need no rescaling, and the 128 threads
            // exchange one bit.
            float arg[ROWS];
            bool exceeds = false;
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (r < nrows) {
                    if (!clear && !(key < kend && key <= pos[r] && key > low[r])) sr[r] = 0xff800000u;   // -inf
                    arg[r] = fmaf(__uint_as_float(sr[r]), sc, -base[r]);     // no reference yet: +inf (NaN for an unseen key)
                    exceeds = exceeds || arg[r] > 8.f;
                }
            }
            bool rescale = false;
            float corr[ROWS];
            if (softmax_meet(exceeds || fail || *(volatile int*)&abort_flag)) {
                // ---- rare: some row's reference point moves (always in a row's first tile)
                if (t < ROWS) ctl.row_max[0][t] = ordered(-INFINITY);
                if (softmax_meet(fail || *(volatile int*)&abort_flag)) { left = true; break; }
                int mine = ordered(-INFINITY);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    if (r < nrows) {
                        const int best = __reduce_max_sync(0xffffffffu, ordered(__uint_as_float(sr[r])));
                        if (lane == r) mine = best;
                    }
                }
                if (lane < nrows) atomicMax(&ctl.row_max[0][lane], mine);    // lane r carries row r
                softmax_meet(false);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    corr[r] = 1.f;
                    if (r < nrows) {
                        const float top = unordered(ctl.row_max[0][r]) * sc;    // the tile's maximum, base-2 units
                        if (top != -INFINITY && (base[r] == -INFINITY || top - base[r] > 8.f)) {
                            if (base[r] == -INFINITY) corr[r] = 0.f;
                            else { corr[r] = fast_exp2(base[r] - top); rescale = true; }
                            base[r] = top;
                            l_run[r] *= corr[r];
                        }
                        arg[r] = fmaf(__uint_as_float(sr[r]), sc, -base[r]);
                    }
                }
            }
            TC_MARK(2);
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (r < nrows) {
                    // a key that the row does not see has score -inf: arg is -inf, or NaN while the
                    // row has no reference point yet; both count as 0
                    const float pr = arg[r] == arg[r] ? fast_exp2(arg[r]) : 0.f;
                    l_run[r] += pr;
                    sr[r] = __float_as_uint(pr);
                }
            }
            TC_MARK(4);
            // P^T and O belong to the tensor core until P V of the tile before has completed
            if (i > 0 && !mbar_wait(&ctl.pv_done, (i - 1) & 1)) fail = true;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            TC_MARK(3);
            if (rescale) {                                   // the same decision in every thread
                uint32_t orr[ROWS];
                tmem_ld16_issue(lane_base + DCOL_O, orr);
                tmem_wait_ld();
#pragma unroll
                for (int r = 0; r < ROWS; ++r) orr[r] = __float_as_uint(__uint_as_float(orr[r]) * corr[r]);
                tmem_st16_issue(lane_base + DCOL_O, orr);
                tmem_wait_st();
            }
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (r < nrows)
                    *reinterpret_cast<bf16*>(p_mine + r * 128 + ((p_chunk ^ (r & 7)) << 4)) = __float2bfloat16_rn(__uint_as_float(sr[r]));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // P^T before the tensor core reads it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            TC_MARK(4);
            mbar_arrive(&ctl.p_ready);
            TC_MARK(5);
        }
        // ---- the last P V, the row sums, then dimension t of every row
        bool have = !left && !fail && ntiles > 0;
        if (have && !mbar_wait(&ctl.pv_done, (ntiles - 1) & 1)) have = false;
        have = __all_sync(0xffffffffu, have);
        if (!have && ntiles > 0 && lane == 0) { atomicExch(x.error, ERR_TCD_SOFTMAX); atomicExch(&abort_flag, 1); }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (r < nrows) {
                const float s = warp_sum(l_run[r]);
                if (lane == 0) ctl.row_sum[quarter][r] = s;
            }
        }
        softmax_meet(false);
        uint32_t orr[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) orr[r] = 0u;
        if (have) { tmem_ld16_issue(lane_base + DCOL_O, orr); tmem_wait_ld(); }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (r < nrows) {
                const float l = (ctl.row_sum[0][r] + ctl.row_sum[1][r]) + (ctl.row_sum[2][r] + ctl.row_sum[3][r]);
                const int row = row0 + r;
                const int tok = qstart + row / group, h = kvh * group + row % group;
                if (p.nsplit == 1) {
                    const float inv = l > 0.f ? 1.0f / l : 0.f;
                    ((bf16*)p.out)[(size_t)tok * p.out_ld + h * HD + t] = __float2bfloat16_rn(__uint_as_float(orr[r]) * inv);
                } else {
                    const size_t idx = ((size_t)split * p.tokens + tok) * p.heads + h;
                    p.part_o[idx * HD + t] = __uint_as_float(orr[r]);
                    if (t == 0) {
                        p.part_ml[idx * 2] = base[r] * 0.6931471805599453f;      // natural units; -inf stays -inf
                        p.part_ml[idx * 2 + 1] = l;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(DTMEM_COLS) : "memory");
    }
}

}  // namespace dec
#endif  // HEAD_DIM == 128

}  // namespace fsie

using namespace fsie;

extern "C" {


int fsie_attn_tc_head_dim() { return HD; }
int fsie_attn_tc_rows() { return STREAMS * BM; }
int fsie_attn_tc_map_bytes() { return (int)sizeof(CUtensorMap); }

// Tensor map of a cache group's pages [num_pages, entries, 2, kv_heads, page_size, head_dim] seen
// as a matrix of head_dim columns; boxes of page_size rows x 64 columns, 128-byte swizzle.
int fsie_attn_tc_pages_map(void* map_out, const void* pages, long long total_rows, int head_dim, int page_size) {
    if (head_dim != HD) return ERR_UNSUPPORTED;
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) return ERR_UNSUPPORTED;
    if (total_rows <= 0 || total_rows >= (1ll << 31)) return ERR_UNSUPPORTED;
    EncodeTiled encode = encode_tiled();
    if (!encode) return ERR_UNSUPPORTED;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)total_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box,
                               elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return ERR_BAD_ARGUMENT;
    memcpy(map_out, &map, sizeof(map));
    return 0;
}

// Tiles of 256 query rows.  Arguments as fsie_attn_mma (attention_mma.cu) without a row class,
// with the pages given as a TMA descriptor (`pages_map`, made by fsie_attn_tc_pages_map over
// `entries` cache entries per page, of which this launch reads `entry`) and the error flag.
int fsie_attn_tc(const void* pages_map, int entries, int entry, const void* q, int q_ld, int page_size,
                 const int* block_tables, int bt_stride, const int* tile_item, const int* tile_row0, int tiles,
                 const int* item_qstart, const int* item_qlen, const int* item_pos0, void* out, int out_ld,
                 float* part_o, float* part_ml, int tokens, int heads, int kv_heads, int head_dim, int window,
                 int nsplit, float scale, const int* combine_tokens, int num_combine, int* error,
                 cudaStream_t stream) {
    if (tiles <= 0 || tokens <= 0) return 0;
    if (head_dim != HD) return ERR_UNSUPPORTED;
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) return ERR_UNSUPPORTED;
    if (kv_heads <= 0 || heads % kv_heads != 0 || nsplit < 1 || nsplit > MAX_KEY_SPLITS || (q_ld % 8) != 0 ||
        (out_ld % 8) != 0 || entries <= 0 || entry < 0 || entry >= entries || !error)
        return ERR_BAD_ARGUMENT;
    if (nsplit > 1 && (!part_o || !part_ml)) return ERR_BAD_ARGUMENT;
    CUtensorMap map;
    memcpy(&map, pages_map, sizeof(map));
    AttnParams p;
    p.q = q; p.q_ld = q_ld; p.k_pages = nullptr; p.v_pages = nullptr;
    p.page_stride = 0; p.page_size = page_size;
    p.block_tables = block_tables; p.bt_stride = bt_stride;
    p.tile_item = tile_item; p.tile_row0 = tile_row0;
    p.item_qstart = item_qstart; p.item_qlen = item_qlen; p.item_pos0 = item_pos0;
    p.out = out; p.out_ld = out_ld; p.part_o = part_o; p.part_ml = part_ml;
    p.tokens = tokens; p.heads = heads; p.kv_heads = kv_heads; p.head_dim = head_dim;
    p.window = window; p.nsplit = nsplit; p.scale = scale;
    TcExtra x;
    x.entries = entries; x.entry = entry; x.error = error;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    attn_tc_kernel<<<dim3(tiles * kv_heads, 1, nsplit), THREADS, SMEM_BYTES, stream>>>(map, p, x);
    int rc = (int)cudaGetLastError();
    if (rc != 0 || nsplit == 1) return rc;
    const int count = combine_tokens ? num_combine : tokens;
    if (count <= 0) return 0;
    attn_combine_kernel<<<dim3(count, heads), HD >= 128 ? 64 : 32, 0, stream>>>(
        part_o, part_ml, (bf16*)out, out_ld, tokens, heads, nsplit, combine_tokens);
    return (int)cudaGetLastError();
}

// Tiles of up to 16 query rows (decoded tokens, two-token portions): attn_tc_decode_kernel.
// Arguments as fsie_attn_tc; head size 128 only (a library built for another head size refuses).
#if HEAD_DIM == 128
int fsie_attn_tc_decode_rows() { return dec::ROWS; }
int fsie_attn_tc_decode(const void* pages_map, int entries, int entry, const void* q, int q_ld, int page_size,
                        const int* block_tables, int bt_stride, const int* tile_item, const int* tile_row0, int tiles,
                        const int* item_qstart, const int* item_qlen, const int* item_pos0, void* out, int out_ld,
                        float* part_o, float* part_ml, int tokens, int heads, int kv_heads, int head_dim, int window,
                        int nsplit, float scale, const int* combine_tokens, int num_combine, int* error,
                        cudaStream_t stream) {
    if (tiles <= 0 || tokens <= 0) return 0;
    if (head_dim != HD || tiles > 65535) return ERR_UNSUPPORTED;     // tiles are the grid's y dimension
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) return ERR_UNSUPPORTED;
    if (kv_heads <= 0 || heads % kv_heads != 0 || nsplit < 1 || nsplit > MAX_KEY_SPLITS || (q_ld % 8) != 0 ||
        entries <= 0 || entry < 0 || entry >= entries || !error)
        return ERR_BAD_ARGUMENT;
    if (nsplit > 1 && (!part_o || !part_ml)) return ERR_BAD_ARGUMENT;
    CUtensorMap map;
    memcpy(&map, pages_map, sizeof(map));
    AttnParams p;
    p.q = q; p.q_ld = q_ld; p.k_pages = nullptr; p.v_pages = nullptr;
    p.page_stride = 0; p.page_size = page_size;
    p.block_tables = block_tables; p.bt_stride = bt_stride;
    p.tile_item = tile_item; p.tile_row0 = tile_row0;
    p.item_qstart = item_qstart; p.item_qlen = item_qlen; p.item_pos0 = item_pos0;
    p.out = out; p.out_ld = out_ld; p.part_o = part_o; p.part_ml = part_ml;
    p.tokens = tokens; p.heads = heads; p.kv_heads = kv_heads; p.head_dim = head_dim;
    p.window = window; p.nsplit = nsplit; p.scale = scale;
    TcExtra x;
    x.entries = entries; x.entry = entry; x.error = error;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(dec::attn_tc_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dec::DSMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    int rc = launch_dependent(dec::attn_tc_decode_kernel, dim3(kv_heads, tiles, nsplit), dim3(dec::DTHREADS),
                              (size_t)dec::DSMEM_BYTES, stream, map, p, x);
    if (rc != 0 || nsplit == 1) return rc;
    const int count = combine_tokens ? num_combine : tokens;
    if (count <= 0) return 0;
    return launch_dependent(attn_combine_kernel, dim3(count, heads), dim3(HD >= 128 ? 64 : 32), 0, stream,
                            (const float*)part_o, (const float*)part_ml, (bf16*)out, out_ld, tokens, heads, nsplit,
                            combine_tokens);
}
#else
int fsie_attn_tc_decode_rows() { return 0; }
int fsie_attn_tc_decode(const void*, int, int, const void*, int, int, const int*, int, const int*, const int*, int,
                        const int*, const int*, const int*, void*, int, float*, float*, int, int, int, int, int, int,
                        float, const int*, int, int*, cudaStream_t) {
    return ERR_UNSUPPORTED;
}
#endif

}  // extern "C"
