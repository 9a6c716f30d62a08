// Causal grouped-query attention over the paged cache, bfloat16, with keys and values fetched
// by the copy engine (TMA).  The arithmetic, the tiling into rows of (token, head) pairs, the
// warp grid and the split of key ranges are those of attention_mma.cu; what differs is how a
// 64-key tile reaches shared memory.  There every thread issues 16-byte cp.async copies and
// all threads meet at a barrier per tile; here a producer warp issues one
// cp.async.bulk.tensor per page and 128-byte column half (the pages of a cache group are one
// 2-D tensor [page x entry x K|V x kv_head x slot, head_dim] to the tensor map), tiles land in
// the 128-byte swizzle that ldmatrix reads without bank conflicts, and producer and consumer
// warps hand stages over through full/empty mbarriers without a block-wide barrier.
// Needs head_dim a multiple of 64 and a page size of 8, 16, 32 or 64; compiled per head size.
//
// Every wait is bounded; when one runs out the kernel sets *error and leaves.
#include "common.cuh"
#include "attention_params.cuh"
#include "tma.cuh"
#include <math.h>
#include <string.h>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
static_assert(HEAD_DIM % 64 == 0 && HEAD_DIM >= 64 && HEAD_DIM <= 256, "head size: 64..256 in steps of 64");

namespace fsie {

constexpr int HD = HEAD_DIM;
constexpr int BN = 64;                 // keys per tile
constexpr int LDS = HD + 8;            // padded row of the query tile (elements)
constexpr int CHUNKS = HD / 8;         // 16-byte chunks per row
constexpr int HALVES = HD / 64;        // 128-byte column halves of a key row
constexpr int HALF_BYTES = BN * 128;   // one column half of a 64-key tile
constexpr int TILE_BYTES = HALVES * HALF_BYTES;
enum { ERR_ATTN_PRODUCER = 41, ERR_ATTN_CONSUMER = 42 };

struct TmaExtra {                      // where a cache entry sits inside its group's page tensor
    int entries, entry, error_slot;    // entries per page, this entry
    int* error;
};

// address of (key, col) inside a tile written by TMA in the 128-byte swizzle (col % 8 == 0)
__device__ __forceinline__ const bf16* tile_at(const unsigned char* tile, int key, int col) {
    const int half = col >> 6, chunk = (col & 63) >> 3;
    return reinterpret_cast<const bf16*>(tile + half * HALF_BYTES + key * 128 + ((chunk ^ (key & 7)) << 4));
}
constexpr bool Q_IN_REGS = HD <= 128;

__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const unsigned d = smem_u32(dst);
    const int bytes = valid ? 16 : 0;          // 0 source bytes: the 16 destination bytes become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
// d += a(16x16, row) * b(16x8, col), bf16 operands, float accumulators
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

}  // namespace fsie
#include "attention_combine.cuh"
namespace fsie {

template <int WARPS_M, int WARPS_K, int STAGES>
struct Shape {
    static constexpr int BM = 16 * WARPS_M;
    static constexpr int KPW = BN / WARPS_K;          // keys of a tile that one warp handles
    static constexpr int NT = KPW / 8;                // 8-key score tiles per warp
    static constexpr int CONSUMERS = 32 * WARPS_M * WARPS_K;
    static constexpr int THREADS = CONSUMERS + 32;     // + the producer warp
    static constexpr size_t Q_BYTES = ((size_t)BM * LDS * sizeof(bf16) + 1023) / 1024 * 1024;
    static constexpr size_t MERGE_BYTES = WARPS_K > 1 ? (size_t)WARPS_K * BM * (HD + 2) * sizeof(float) : 0;
    static constexpr size_t PIPE_BYTES = 2 * (size_t)STAGES * TILE_BYTES;
    static constexpr size_t SMEM = 1024 + Q_BYTES + (PIPE_BYTES > MERGE_BYTES ? PIPE_BYTES : MERGE_BYTES);
};

template <int WARPS_M, int WARPS_K, int STAGES>
__global__ void __launch_bounds__(32 * WARPS_M * WARPS_K + 32, 2)
attn_tma_kernel(const __grid_constant__ CUtensorMap pages_map, const AttnParams p, const TmaExtra x) {
    using S = Shape<WARPS_M, WARPS_K, STAGES>;
    constexpr int BM = S::BM, KPW = S::KPW, NT = S::NT, THREADS = S::THREADS, CONSUMERS = S::CONSUMERS;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem_raw = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    unsigned char* Ks = smem_raw + S::Q_BYTES;                 // [STAGES][TILE_BYTES], 1,024-aligned
    unsigned char* Vs = Ks + (size_t)STAGES * TILE_BYTES;
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES];

    // blocks start in the order of blockIdx.x: all kv heads of a tile, then the next tile (the
    // caller lists the tiles that see the most keys first)
    const int kvh = blockIdx.x, tile = blockIdx.y, split = blockIdx.z;
    const int group = p.heads / p.kv_heads;
    const int item = p.tile_item[tile];
    const int row0 = p.tile_row0[tile];
    const int qstart = p.item_qstart[item], qlen = p.item_qlen[item], pos0 = p.item_pos0[item];
    const int nrows = min(BM, qlen * group - row0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp / WARPS_K, wk = warp % WARPS_K;
    const int g = lane >> 2, t = lane & 3;
    const bf16* q = (const bf16*)p.q;
    const int* bt = p.block_tables + (size_t)item * p.bt_stride;

    // key range of the tile (see attention_generic.cu)
    const int pos_first = pos0 + row0 / group;
    const int pos_last = pos0 + (row0 + nrows - 1) / group;
    int kbegin = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    int kend = pos_last + 1;
    if (p.nsplit > 1) {
        const int span = kend - kbegin;
        int chunk = (span + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + BN - 1) / BN) * BN;
        const int b = kbegin + split * chunk;
        kend = min(kend, b + chunk);
        kbegin = b;
    }
    kbegin = kbegin / BN * BN;        // tiles hold whole pages; keys before the window are masked anyway
    const int ntiles = kend > kbegin ? (kend - kbegin + BN - 1) / BN : 0;

    // ---- stage the query rows (rows beyond the tile's count are zero); clear the stages once so
    // that pages which are never fetched (beyond the range, or given back) read as finite numbers
    for (int e = tid; e < BM * CHUNKS; e += THREADS) {
        const int r = e / CHUNKS, c = e - r * CHUNKS;
        const bool ok = r < nrows;
        const int row = row0 + (ok ? r : 0);
        const int tok = qstart + row / group, h = kvh * group + row % group;
        cp_async16(Qs + r * LDS + c * 8, q + (size_t)tok * p.q_ld + h * HD + c * 8, ok);
    }
    cp_async_commit();
    for (int e = tid; e < 2 * STAGES * TILE_BYTES / 16; e += THREADS)
        reinterpret_cast<uint4*>(Ks)[e] = make_uint4(0, 0, 0, 0);
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], WARPS_M * WARPS_K); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    cp_async_wait<0>();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeros precede the copy engine's writes
    __syncthreads();

    if (warp == WARPS_M * WARPS_K) {
        // ------------------------------------------------------------------ producer warp
        // lane j looks up and fetches page j of the tile: the table reads and the copy
        // instructions of a tile go out side by side instead of one after the other
        const int ps = p.page_size, pages_per_tile = BN / ps;
        // rows of the [all pages x entries x K|V x kv heads x slots, head_dim] tensor
        const long long rows_per_page = (long long)x.entries * 2 * p.kv_heads * ps;
        const long long k_row0 = ((long long)x.entry * 2) * p.kv_heads * ps + (long long)kvh * ps;
        const long long v_row0 = k_row0 + (long long)p.kv_heads * ps;
        for (int i = 0; i < ntiles; ++i) {
            const int s = i % STAGES;
            const int key = kbegin + i * BN + lane * ps;
            const int page = (lane < pages_per_tile && key < kend) ? bt[key / ps] : -1;
            bool ok = true;
            if (lane == 0 && i >= STAGES) ok = mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0) atomicExch(x.error, ERR_ATTN_PRODUCER);
                break;
            }
            const int wanted = __popc(__ballot_sync(0xffffffffu, page >= 0));
            if (lane == 0) mbar_expect_tx(&full_bar[s], (uint32_t)wanted * ps * HD * 2 * 2);
            __syncwarp();
            if (page >= 0) {
                unsigned char* kd = Ks + (size_t)s * TILE_BYTES + lane * ps * 128;
                unsigned char* vd = Vs + (size_t)s * TILE_BYTES + lane * ps * 128;
                const long long base = (long long)page * rows_per_page;
#pragma unroll
                for (int h = 0; h < HALVES; ++h) {
                    tma_load_2d(kd + h * HALF_BYTES, &pages_map, h * 64, (int)(base + k_row0), &full_bar[s]);
                    tma_load_2d(vd + h * HALF_BYTES, &pages_map, h * 64, (int)(base + v_row0), &full_bar[s]);
                }
            }
        }
        return;
    }

    // ---- per-thread state: rows g and g+8 of the warp's 16 rows
    const int r_lo = wm * 16 + g, r_hi = r_lo + 8;
    const int pos_lo = r_lo < nrows ? pos0 + (row0 + r_lo) / group : -1;   // -1: sees no key
    const int pos_hi = r_hi < nrows ? pos0 + (row0 + r_hi) / group : -1;
    const int lowest_lo = p.window > 0 ? pos_lo - p.window : -1;           // keys <= this are unseen
    const int lowest_hi = p.window > 0 ? pos_hi - p.window : -1;
    const float sc = p.scale * 1.4426950408889634f;                        // scores in base-2 units
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }

    unsigned qf[Q_IN_REGS ? HD / 16 : 1][4];
    const bf16* q_ld_addr = Qs + (wm * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + 8 * (lane >> 4);

    if (Q_IN_REGS) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) ldmatrix_x4(qf[ks], q_ld_addr + ks * 16);
    }
    bool alive = true;
    for (int i = 0; i < ntiles && alive; ++i) {
        const int stage = i % STAGES;
        if (!mbar_wait(&full_bar[stage], (i / STAGES) & 1)) {
            if (lane == 0) atomicExch(x.error, ERR_ATTN_CONSUMER);
            alive = false;
            break;
        }
        // every exit from this iteration hands the stage back to the producer
        struct Release {
            uint64_t* bar; int lane;
            __device__ ~Release() { __syncwarp(); if (lane == 0) mbar_arrive(bar); }
        } release{&empty_bar[stage], lane};
        const int k0 = kbegin + i * BN + wk * KPW;          // first key of this warp in the tile
        const bool future = k0 > max(pos_lo, pos_hi);     // beyond what this thread's rows see
        if (k0 >= kend || __all_sync(0xffffffffu, future))
            continue;                                        // nothing visible for this warp
        const unsigned char* kt = Ks + (size_t)stage * TILE_BYTES;
        const unsigned char* vt = Vs + (size_t)stage * TILE_BYTES;
        const int key0 = wk * KPW;                           // this warp's first key inside the tile

        // ---- scores S[16 rows, KPW keys] = Q K^T
        float s[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            unsigned a[4];
            if (Q_IN_REGS) { a[0] = qf[ks][0]; a[1] = qf[ks][1]; a[2] = qf[ks][2]; a[3] = qf[ks][3]; }
            else ldmatrix_x4(a, q_ld_addr + ks * 16);
#pragma unroll
            for (int n2 = 0; n2 < NT / 2; ++n2) {
                unsigned b[4];
                ldmatrix_x4(b, tile_at(kt, key0 + n2 * 16 + (lane & 7) + 8 * (lane >> 4), ks * 16 + 8 * ((lane >> 3) & 1)));
                mma_bf16(s[2 * n2], a, b[0], b[1]);
                mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
            }
        }
        // ---- mask (only where some key of this warp's range is hidden from some row), maximum
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
        const int k_last = k0 + KPW - 1;
        // rows beyond the tile's count are never written: they do not force the masked path
        const int see_lo = r_lo < nrows ? pos_lo : 0x7fffffff, see_hi = r_hi < nrows ? pos_hi : 0x7fffffff;
        const bool clear = k_last < kend && k_last <= min(see_lo, see_hi) &&
                           k0 > max(lowest_lo, lowest_hi);
        if (__all_sync(0xffffffffu, clear)) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                mx_lo = fmaxf(mx_lo, fmaxf(s[n][0], s[n][1]));
                mx_hi = fmaxf(mx_hi, fmaxf(s[n][2], s[n][3]));
            }
        } else {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = k0 + n * 8 + 2 * t + e;
                    const bool in = key < kend;
                    if (!(in && key <= pos_lo && key > lowest_lo)) s[n][e] = -INFINITY;
                    if (!(in && key <= pos_hi && key > lowest_hi)) s[n][2 + e] = -INFINITY;
                    mx_lo = fmaxf(mx_lo, s[n][e]);
                    mx_hi = fmaxf(mx_hi, s[n][2 + e]);
                }
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo * sc;     // avoid inf - inf
        const float base_hi = mn_hi == -INFINITY ? 0.f : mn_hi * sc;
        const float corr_lo = exp2f(m_lo * sc - base_lo), corr_hi = exp2f(m_hi * sc - base_hi);
        m_lo = mn_lo; m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            s[n][0] = exp2f(s[n][0] * sc - base_lo); s[n][1] = exp2f(s[n][1] * sc - base_lo);
            s[n][2] = exp2f(s[n][2] * sc - base_hi); s[n][3] = exp2f(s[n][3] * sc - base_hi);
            sum_lo += s[n][0] + s[n][1];
            sum_hi += s[n][2] + s[n][3];
        }
        l_lo = l_lo * corr_lo + sum_lo;          // per-thread partial; the quad is summed at the end
        l_hi = l_hi * corr_hi + sum_hi;
        if (__any_sync(0xffffffffu, corr_lo != 1.f || corr_hi != 1.f)) {
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                o[n][0] *= corr_lo; o[n][1] *= corr_lo; o[n][2] *= corr_hi; o[n][3] *= corr_hi;
            }
        }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < KPW / 16; ++kk) {
            unsigned a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int d2 = 0; d2 < HD / 16; ++d2) {
                unsigned b[4];
                ldmatrix_x4_trans(b, tile_at(vt, key0 + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), d2 * 16 + 8 * (lane >> 4)));
                mma_bf16(o[2 * d2], a, b[0], b[1]);
                mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
            }
        }
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    // maxima in natural units of the scaled scores, as the merge kernels expect
    float mnat_lo = m_lo == -INFINITY ? -INFINITY : m_lo * p.scale;
    float mnat_hi = m_hi == -INFINITY ? -INFINITY : m_hi * p.scale;

    if constexpr (WARPS_K > 1) {
        // ---- merge the WARPS_K partial results of each row through shared memory
        // every consumer warp is done with the pipeline (the producer warp has left: a named
        // barrier over the consumers only)
        asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory");
        float* Om = reinterpret_cast<float*>(smem_raw + S::Q_BYTES);          // [WARPS_K][BM][HD]
        float* Mm = Om + (size_t)WARPS_K * BM * HD;                           // [WARPS_K][BM]
        float* Lm = Mm + WARPS_K * BM;                                        // [WARPS_K][BM]
        float* ow = Om + ((size_t)wk * BM) * HD;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            *reinterpret_cast<float2*>(ow + r_lo * HD + n * 8 + 2 * t) = make_float2(o[n][0], o[n][1]);
            *reinterpret_cast<float2*>(ow + r_hi * HD + n * 8 + 2 * t) = make_float2(o[n][2], o[n][3]);
        }
        if (t == 0) {
            Mm[wk * BM + r_lo] = mnat_lo; Lm[wk * BM + r_lo] = l_lo;
            Mm[wk * BM + r_hi] = mnat_hi; Lm[wk * BM + r_hi] = l_hi;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory");
        for (int e = tid; e < nrows * (HD / 2); e += CONSUMERS) {
            const int r = e / (HD / 2), d = (e - r * (HD / 2)) * 2;
            float mm = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS_K; ++w) mm = fmaxf(mm, Mm[w * BM + r]);
            float l = 0.f, a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS_K; ++w) {
                const float mw = Mm[w * BM + r];
                if (mw == -INFINITY) continue;
                const float f = __expf(mw - mm);
                l += Lm[w * BM + r] * f;
                const float2 v = *reinterpret_cast<const float2*>(Om + ((size_t)w * BM + r) * HD + d);
                a0 += v.x * f; a1 += v.y * f;
            }
            const int row = row0 + r;
            const int tok = qstart + row / group, h = kvh * group + row % group;
            if (p.nsplit == 1) {
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                *reinterpret_cast<__nv_bfloat162*>((bf16*)p.out + (size_t)tok * p.out_ld + h * HD + d) =
                    __floats2bfloat162_rn(a0 * inv, a1 * inv);
            } else {
                const size_t idx = ((size_t)split * p.tokens + tok) * p.heads + h;
                *reinterpret_cast<float2*>(p.part_o + idx * HD + d) = make_float2(a0, a1);
                if (d == 0) { p.part_ml[idx * 2] = mm; p.part_ml[idx * 2 + 1] = l; }
            }
        }
    } else {
    // ---- WARPS_K == 1: write straight from the accumulators
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = half ? r_hi : r_lo;
        if (r >= nrows) continue;
        const float l = half ? l_hi : l_lo;
        const float mnat = half ? mnat_hi : mnat_lo;
        const int row = row0 + r;
        const int tok = qstart + row / group, h = kvh * group + row % group;
        if (p.nsplit == 1) {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = (bf16*)p.out + (size_t)tok * p.out_ld + h * HD;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n)
                *reinterpret_cast<__nv_bfloat162*>(dst + n * 8 + 2 * t) =
                    __floats2bfloat162_rn(o[n][2 * half] * inv, o[n][2 * half + 1] * inv);
        } else {
            const size_t idx = ((size_t)split * p.tokens + tok) * p.heads + h;
            float* dst = p.part_o + idx * HD;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n)
                *reinterpret_cast<float2*>(dst + n * 8 + 2 * t) = make_float2(o[n][2 * half], o[n][2 * half + 1]);
            if (t == 0) { p.part_ml[idx * 2] = mnat; p.part_ml[idx * 2 + 1] = l; }
        }
    }
    }
}

template <int WARPS_M, int WARPS_K, int STAGES>
static int launch(const CUtensorMap& map, const AttnParams& p, const TmaExtra& x, int tiles, cudaStream_t stream) {
    using S = Shape<WARPS_M, WARPS_K, STAGES>;
    auto kernel = attn_tma_kernel<WARPS_M, WARPS_K, STAGES>;
    static bool configured = false;            // per process and kernel; harmless if repeated
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(p.kv_heads, tiles, p.nsplit);
    kernel<<<grid, S::THREADS, S::SMEM, stream>>>(map, p, x);
    return (int)cudaGetLastError();
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_attn_tma_head_dim() { return HD; }
int fsie_attn_tma_map_bytes() { return (int)sizeof(CUtensorMap); }

// Tensor map of one cache group's pages [num_pages, entries, 2, kv_heads, page_size, head_dim]
// (bfloat16, contiguous) seen as a matrix of head_dim columns; boxes of page_size rows x 64 columns.
int fsie_attn_tma_pages_map(void* map_out, const void* pages, long long total_rows, int head_dim, int page_size) {
    if (head_dim != HD) return ERR_UNSUPPORTED;
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return ERR_UNSUPPORTED;
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

// As fsie_attn_mma (attention_mma.cu), with the group's tensor map and the place of this cache
// entry in it (entries per page, index of the entry) instead of key and value base pointers.
int fsie_attn_tma(int row_class, const void* pages_map, int entries, int entry, const void* q, int q_ld,
                  int page_size, const int* block_tables, int bt_stride,
                  const int* tile_item, const int* tile_row0, int tiles, const int* item_qstart,
                  const int* item_qlen, const int* item_pos0, void* out, int out_ld, float* part_o,
                  float* part_ml, int tokens, int heads, int kv_heads, int head_dim, int window,
                  int nsplit, float scale, const int* combine_tokens, int num_combine, int* error,
                  cudaStream_t stream) {
    if (tiles <= 0 || tokens <= 0) return 0;
    if (tiles > 65535) return ERR_UNSUPPORTED;          // tiles are the grid's y dimension
    if (head_dim != HD) return ERR_UNSUPPORTED;
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return ERR_UNSUPPORTED;
    if (kv_heads <= 0 || heads % kv_heads != 0 || nsplit < 1 || nsplit > 32 || (q_ld % 8) != 0 ||
        (out_ld % 2) != 0 || entries <= 0 || entry < 0 || entry >= entries || !error)
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
    TmaExtra x;
    x.entries = entries; x.entry = entry; x.error_slot = 0; x.error = error;
    int rc;
    if (row_class == 0) rc = launch<1, 4, 2>(map, p, x, tiles, stream);
    else if (row_class == 1) rc = launch<2, 2, 3>(map, p, x, tiles, stream);
    else rc = launch<4, 1, 2>(map, p, x, tiles, stream);
    if (rc != 0 || nsplit == 1) return rc;
    const int count = combine_tokens ? num_combine : tokens;
    if (count <= 0) return 0;
    dim3 cgrid(count, heads);
    attn_combine_kernel<<<cgrid, HD >= 128 ? 64 : 32, 0, stream>>>(
        part_o, part_ml, (bf16*)out, out_ld, tokens, heads, nsplit, combine_tokens);
    return (int)cudaGetLastError();
}

}  // extern "C"
