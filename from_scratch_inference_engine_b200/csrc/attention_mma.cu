// Causal grouped-query attention over the paged cache on the tensor cores, bfloat16 storage,
// 32-bit scores, softmax statistics and accumulation.  Compiled once per head size
// (-DHEAD_DIM=N, a multiple of 16 up to 256) when a model with that head size is loaded.
//
// Same tiling as attention_generic.cu: a tile is BM query rows of one request and one kv
// head, a row being a (new token, query head of the group) pair, so the heads of a group
// share every key/value tile and a prompt portion and a decoded token differ only in the
// number of rows.  Keys and values arrive in tiles of 64 keys through a cp.async pipeline
// (16-byte copies straight from the pages, page by page through the block table).
//
// The block's warps form a WARPS_M x WARPS_K grid: warp (wm, wk) owns rows 16*wm..16*wm+15
// and, inside every 64-key tile, the keys wk*(64/WARPS_K).. - each warp keeps its own
// running softmax over its keys and the WARPS_K results are merged through shared memory at
// the end.  Prompt portions use 4x1 (64 rows), a single decoded token with a group of up to
// 16 heads uses 1x4: all four warps stream keys for the same 16 rows.
// The key range of a tile may also be split over blockIdx.z; attn_combine merges those.
//
// Formula: src/model/nn.cpp:151-226 of the reference (scores (q.k)/sqrt(d) over keys
// 0..position, softmax, weighted sum of values), as a running softmax.
#include "common.cuh"
#include "attention_params.cuh"
#include <math.h>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head size: 16..256 in steps of 16");

namespace fsie {

constexpr int HD = HEAD_DIM;
constexpr int BN = 64;                 // keys per tile
constexpr int LDS = HD + 8;            // padded row of a shared tile (elements): conflict-free ldmatrix
constexpr int CHUNKS = HD / 8;         // 16-byte chunks per row
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
    static constexpr int THREADS = 32 * WARPS_M * WARPS_K;
    static constexpr size_t TILE_BYTES = (size_t)BN * LDS * sizeof(bf16);
    static constexpr size_t Q_BYTES = (size_t)BM * LDS * sizeof(bf16);
    static constexpr size_t MERGE_BYTES = WARPS_K > 1 ? (size_t)WARPS_K * BM * (HD + 2) * sizeof(float) : 0;
    static constexpr size_t PIPE_BYTES = 2 * STAGES * TILE_BYTES;
    static constexpr size_t SMEM = Q_BYTES + (PIPE_BYTES > MERGE_BYTES ? PIPE_BYTES : MERGE_BYTES);
};

template <int WARPS_M, int WARPS_K, int STAGES>
__global__ void __launch_bounds__(32 * WARPS_M * WARPS_K)
attn_mma_kernel(const AttnParams p) {
    using S = Shape<WARPS_M, WARPS_K, STAGES>;
    constexpr int BM = S::BM, KPW = S::KPW, NT = S::NT, THREADS = S::THREADS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = reinterpret_cast<bf16*>(smem_raw + S::Q_BYTES);
    bf16* Vs = Ks + (size_t)STAGES * BN * LDS;

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
    const bf16* kp = (const bf16*)p.k_pages;
    const bf16* vp = (const bf16*)p.v_pages;
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
    const int ntiles = kend > kbegin ? (kend - kbegin + BN - 1) / BN : 0;

    // Element offset of every key row of a tile inside the pages (-1: not to be read), worked
    // out one loop iteration before the tile is fetched, so that the fetch itself is a
    // shared-memory read and two 16-byte copies per thread and pass, all coalesced.
    __shared__ long long key_base[STAGES][BN];
    auto find_rows = [&](int stage, int k0) {
        if (tid < BN) {
            const int kj = k0 + tid;
            long long base = -1;
            if (kj < kend) {
                const int block = kj / p.page_size;
                const int page = bt[block];
                if (page >= 0)
                    base = (long long)page * p.page_stride +
                           ((long long)kvh * p.page_size + (kj - block * p.page_size)) * HD;
            }
            key_base[stage][tid] = base;
        }
    };
    auto load_tile = [&](int stage) {
        bf16* kd = Ks + (size_t)stage * BN * LDS;
        bf16* vd = Vs + (size_t)stage * BN * LDS;
#pragma unroll 4
        for (int e = tid; e < BN * CHUNKS; e += THREADS) {
            const int j = e / CHUNKS, c = e - j * CHUNKS;
            const long long base = key_base[stage][j];
            const bool ok = base >= 0;
            const long long src = (ok ? base : 0) + c * 8;
            cp_async16(kd + j * LDS + c * 8, kp + src, ok);
            cp_async16(vd + j * LDS + c * 8, vp + src, ok);
        }
    };

#pragma unroll
    for (int s = 0; s < STAGES; ++s) find_rows(s, kbegin + s * BN);
    __syncthreads();
    // Under programmatic dependent launch the kernel before this one (which writes this step's
    // new keys, values and rotated queries) may still be running.  The lists and block tables
    // read so far were staged before the step; keys older than every new token of the request
    // were written by earlier steps: a first tile of only such keys is asked for at once.
    const bool early = ntiles > 0 && kbegin + BN <= pos0;
    if (early) load_tile(0);
    cp_async_commit();
    grid_dependency_wait();
    grid_dependents_go();
    // ---- stage the query rows (rows beyond the tile's count are zero)
    for (int e = tid; e < BM * CHUNKS; e += THREADS) {
        const int r = e / CHUNKS, c = e - r * CHUNKS;
        const bool ok = r < nrows;
        const int row = row0 + (ok ? r : 0);
        const int tok = qstart + row / group, h = kvh * group + row % group;
        cp_async16(Qs + r * LDS + c * 8, q + (size_t)tok * p.q_ld + h * HD + c * 8, ok);
    }
    if (!early && ntiles > 0) load_tile(0);
    cp_async_commit();
#pragma unroll
    for (int s = 1; s < STAGES - 1; ++s) {
        if (s < ntiles) load_tile(s);
        cp_async_commit();
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

    for (int i = 0; i < ntiles; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (i + STAGES - 1 < ntiles) load_tile((i + STAGES - 1) % STAGES);
        cp_async_commit();
        if (i + STAGES < ntiles) find_rows(i % STAGES, kbegin + (i + STAGES) * BN);   // read next round
        if (Q_IN_REGS && i == 0) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) ldmatrix_x4(qf[ks], q_ld_addr + ks * 16);
        }
        const int stage = i % STAGES;
        const int k0 = kbegin + i * BN + wk * KPW;          // first key of this warp in the tile
        const bool future = k0 > max(pos_lo, pos_hi);     // beyond what this thread's rows see
        if (k0 >= kend || __all_sync(0xffffffffu, future))
            continue;                                        // nothing visible for this warp
        const bf16* kt = Ks + (size_t)stage * BN * LDS + (wk * KPW) * LDS;
        const bf16* vt = Vs + (size_t)stage * BN * LDS + (wk * KPW) * LDS;

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
                ldmatrix_x4(b, kt + (n2 * 16 + (lane & 7) + 8 * (lane >> 4)) * LDS + ks * 16 + 8 * ((lane >> 3) & 1));
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
                ldmatrix_x4_trans(b, vt + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + d2 * 16 + 8 * (lane >> 4));
                mma_bf16(o[2 * d2], a, b[0], b[1]);
                mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    // maxima in natural units of the scaled scores, as the merge kernels expect
    float mnat_lo = m_lo == -INFINITY ? -INFINITY : m_lo * p.scale;
    float mnat_hi = m_hi == -INFINITY ? -INFINITY : m_hi * p.scale;

    if constexpr (WARPS_K > 1) {
        // ---- merge the WARPS_K partial results of each row through shared memory
        __syncthreads();                                   // every warp is done with the pipeline
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
        __syncthreads();
        for (int e = tid; e < nrows * (HD / 2); e += THREADS) {
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
static int launch(const AttnParams& p, int tiles, cudaStream_t stream) {
    using S = Shape<WARPS_M, WARPS_K, STAGES>;
    auto kernel = attn_mma_kernel<WARPS_M, WARPS_K, STAGES>;
    static bool configured = false;            // per process and kernel; harmless if repeated
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(p.kv_heads, tiles, p.nsplit);
    return launch_dependent(kernel, grid, dim3(S::THREADS), S::SMEM, stream, p);
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_attn_mma_head_dim() { return HD; }

// rows per tile of a row class: 0 -> 16 rows (1x4 warps), 1 -> 32 rows (2x2), 2 -> 64 rows (4x1)
int fsie_attn_mma_rows(int row_class) { return row_class == 0 ? 16 : (row_class == 1 ? 32 : 64); }

// Launch one row class over its tiles.  With nsplit > 1 the caller provides part_o
// [nsplit, tokens, heads, head_dim] and part_ml [nsplit, tokens, heads, 2] (float), and
// `combine_tokens` (count `num_combine`) lists the tokens of this class whose splits are merged
// (nullptr = all tokens).
int fsie_attn_mma(int row_class, const void* q, int q_ld, const void* k_pages, const void* v_pages,
                  long long page_stride, int page_size, const int* block_tables, int bt_stride,
                  const int* tile_item, const int* tile_row0, int tiles, const int* item_qstart,
                  const int* item_qlen, const int* item_pos0, void* out, int out_ld, float* part_o,
                  float* part_ml, int tokens, int heads, int kv_heads, int head_dim, int window,
                  int nsplit, float scale, const int* combine_tokens, int num_combine,
                  cudaStream_t stream) {
    if (tiles <= 0 || tokens <= 0) return 0;
    if (tiles > 65535) return ERR_UNSUPPORTED;          // tiles are the grid's y dimension
    if (head_dim != HD) return ERR_UNSUPPORTED;
    if (kv_heads <= 0 || heads % kv_heads != 0 || nsplit < 1 || page_size <= 0 || (q_ld % 8) != 0 ||
        (out_ld % 2) != 0 || (page_stride % 8) != 0)
        return ERR_BAD_ARGUMENT;
    if (nsplit > 1 && (!part_o || !part_ml)) return ERR_BAD_ARGUMENT;
    AttnParams p;
    p.q = q; p.q_ld = q_ld; p.k_pages = k_pages; p.v_pages = v_pages;
    p.page_stride = page_stride; p.page_size = page_size;
    p.block_tables = block_tables; p.bt_stride = bt_stride;
    p.tile_item = tile_item; p.tile_row0 = tile_row0;
    p.item_qstart = item_qstart; p.item_qlen = item_qlen; p.item_pos0 = item_pos0;
    p.out = out; p.out_ld = out_ld; p.part_o = part_o; p.part_ml = part_ml;
    p.tokens = tokens; p.heads = heads; p.kv_heads = kv_heads; p.head_dim = head_dim;
    p.window = window; p.nsplit = nsplit; p.scale = scale;
    int rc;
    // two stages for decoded tokens: three blocks fit on an SM, and the kernel is bound by the
    // latency of each block's tile-after-tile chain, not by bytes in flight (measured: 2 stages
    // 118 us, 3 stages 136 us, 4 stages 202 us at batch 64, context 4,096)
    if (row_class == 0) rc = launch<1, 4, 2>(p, tiles, stream);
    else if (row_class == 1) rc = launch<2, 2, 3>(p, tiles, stream);
    else rc = launch<4, 1, 2>(p, tiles, stream);
    if (rc != 0 || nsplit == 1) return rc;
    const int count = combine_tokens ? num_combine : tokens;
    if (count <= 0) return 0;
    dim3 cgrid(count, heads);
    if (nsplit > MAX_KEY_SPLITS) return ERR_BAD_ARGUMENT;
    return launch_dependent(attn_combine_kernel, cgrid, dim3(HD >= 128 ? 64 : 32), 0, stream,
                            (const float*)part_o, (const float*)part_ml, (bf16*)out, out_ld, tokens, heads, nsplit,
                            combine_tokens);
}

}  // extern "C"
