// Causal grouped-query attention over the paged cache, for any head size, group size
// and page size, in 32-bit arithmetic on CUDA cores.  It is the attention of the
// float32 path (storage float) and the fallback of the bfloat16 path (storage bf16)
// for head sizes the tensor-core kernel does not take.
//
// Work is cut into tiles of ROWS query rows of one request and one kv head, where a
// row is a (new token, query head of the group) pair: row = token * group + g.  So a
// prompt portion and a single decoded token are the same case with different row
// counts, and all heads of a group share each key/value tile.  A tile's key range may
// be split over blockIdx.z; split results are merged by attn_combine_kernel.
//
// Mathematics as the reference's attention (src/model/nn.cpp:151-226): scores
// (q.k)/sqrt(head_dim) over keys 0..position (inclusive, optionally only the last
// `window` of them), softmax, weighted sum of values; here as a running softmax in
// 32-bit like the reference GPU kernel does in 64-bit (src/cuda/device.cu:139-190).
#include "common.cuh"
#include "attention_params.cuh"
#include <math.h>

namespace fsie {

constexpr int ROWS = 32;          // query rows per tile
constexpr int WARPS = 8;          // warps per block; each owns ROWS / WARPS rows
constexpr int RPW = ROWS / WARPS;
constexpr int KT = 32;            // keys per shared-memory tile (one per lane)
constexpr int MAX_DPL = 8;        // head_dim <= 32 * MAX_DPL


template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_generic_kernel(const AttnParams p) {
    extern __shared__ float smem[];
    const int hd = p.head_dim;
    float* qs = smem;                         // [ROWS][hd]
    float* ks = qs + ROWS * hd;               // [KT][hd + 1]
    float* vs = ks + KT * (hd + 1);           // [KT][hd]
    __shared__ long long key_base[KT];

    // blocks start in the order of blockIdx.x: all kv heads of a tile, then the next tile (the
    // caller lists the tiles that see the most keys first)
    const int kvh = blockIdx.x, tile = blockIdx.y, split = blockIdx.z;
    const int group = p.heads / p.kv_heads;
    const int item = p.tile_item[tile];
    const int row0 = p.tile_row0[tile];
    const int qstart = p.item_qstart[item], qlen = p.item_qlen[item], pos0 = p.item_pos0[item];
    const int nrows = min(ROWS, qlen * group - row0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* q = (const T*)p.q;
    const T* kp = (const T*)p.k_pages;
    const T* vp = (const T*)p.v_pages;
    const int* bt = p.block_tables + (size_t)item * p.bt_stride;

    // stage the tile's query rows, pre-multiplied by the scale
    for (int e = tid; e < nrows * hd; e += blockDim.x) {
        const int r = e / hd, d = e - r * hd;
        const int row = row0 + r;
        const int tok = qstart + row / group, h = kvh * group + row % group;
        qs[r * hd + d] = to_float(q[(size_t)tok * p.q_ld + h * hd + d]) * p.scale;
    }

    // key range of the tile: up to the last row's position, from the first row's window start
    const int pos_first = pos0 + row0 / group;
    const int pos_last = pos0 + (row0 + nrows - 1) / group;
    int kbegin = 0;
    if (p.window > 0) kbegin = max(0, pos_first - p.window + 1);
    int kend = pos_last + 1;
    if (p.nsplit > 1) {
        const int span = kend - kbegin;
        int chunk = (span + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + KT - 1) / KT) * KT;
        const int b = kbegin + split * chunk;
        kend = min(kend, b + chunk);
        kbegin = b;
    }

    float m[RPW], l[RPW], acc[RPW][MAX_DPL];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < MAX_DPL; ++c) acc[i][c] = 0.f;
    }

    for (int k0 = kbegin; k0 < kend; k0 += KT) {
        __syncthreads();   // previous tile fully consumed (and qs staged, first time)
        if (tid < KT) {
            const int kj = k0 + tid;
            long long base = -1;
            if (kj < kend) {
                const int page = bt[kj / p.page_size];
                if (page >= 0)
                    base = (long long)page * p.page_stride +
                           ((long long)kvh * p.page_size + kj % p.page_size) * hd;
            }
            key_base[tid] = base;
        }
        __syncthreads();
        for (int e = tid; e < KT * hd; e += blockDim.x) {
            const int j = e / hd, d = e - j * hd;
            const long long base = key_base[j];
            ks[j * (hd + 1) + d] = base >= 0 ? to_float(kp[base + d]) : 0.f;
            vs[j * hd + d] = base >= 0 ? to_float(vp[base + d]) : 0.f;
        }
        __syncthreads();
        const int kj = k0 + lane;
        const bool key_ok = kj < kend && key_base[lane] >= 0;
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = warp * RPW + i;
            if (r >= nrows) continue;                 // uniform per warp
            const int pos = pos0 + (row0 + r) / group;
            if (k0 > pos) continue;                   // whole tile is in this row's future
            const bool seen = key_ok && kj <= pos && (p.window <= 0 || kj > pos - p.window);
            float s = 0.f;
            const float* qr = qs + r * hd;
            const float* kr = ks + lane * (hd + 1);
            for (int d = 0; d < hd; ++d) s = fmaf(qr[d], kr[d], s);
            s = seen ? s : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(s));
            if (m_new == -INFINITY) continue;         // nothing visible yet
            const float corr = expf(m[i] - m_new);  // m[i] = -inf gives 0
            const float pj = seen ? expf(s - m_new) : 0.f;
            l[i] = l[i] * corr + warp_sum(pj);
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < MAX_DPL; ++c) acc[i][c] *= corr;
            for (int j = 0; j < KT; ++j) {
                const float pw = __shfl_sync(0xffffffffu, pj, j);
                const float* vr = vs + j * hd;
#pragma unroll
                for (int c = 0; c < MAX_DPL; ++c) {
                    const int d = lane + 32 * c;
                    if (d < hd) acc[i][c] = fmaf(pw, vr[d], acc[i][c]);
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp * RPW + i;
        if (r >= nrows) continue;
        const int row = row0 + r;
        const int tok = qstart + row / group, h = kvh * group + row % group;
        if (p.nsplit == 1) {
            T* o = (T*)p.out + (size_t)tok * p.out_ld + h * hd;
            const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
            for (int c = 0; c < MAX_DPL; ++c) {
                const int d = lane + 32 * c;
                if (d < hd) o[d] = from_float<T>(acc[i][c] * inv);
            }
        } else {
            const size_t idx = ((size_t)split * p.tokens + tok) * p.heads + h;
            float* o = p.part_o + idx * hd;
#pragma unroll
            for (int c = 0; c < MAX_DPL; ++c) {
                const int d = lane + 32 * c;
                if (d < hd) o[d] = acc[i][c];
            }
            if (lane == 0) { p.part_ml[idx * 2] = m[i]; p.part_ml[idx * 2 + 1] = l[i]; }
        }
    }
}

// Merge the splits of one (token, head): o = sum_z acc_z e^(m_z - M) / sum_z l_z e^(m_z - M).
template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, T* __restrict__ out,
                                    int out_ld, int tokens, int heads, int hd, int nsplit) {
    const int tok = blockIdx.x, h = blockIdx.y;
    float mmax = -INFINITY;
    for (int z = 0; z < nsplit; ++z)
        mmax = fmaxf(mmax, part_ml[(((size_t)z * tokens + tok) * heads + h) * 2]);
    float denom = 0.f;
    for (int z = 0; z < nsplit; ++z) {
        const size_t idx = ((size_t)z * tokens + tok) * heads + h;
        const float mz = part_ml[idx * 2];
        if (mz != -INFINITY) denom += part_ml[idx * 2 + 1] * expf(mz - mmax);
    }
    const float inv = denom > 0.f ? 1.0f / denom : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
        for (int z = 0; z < nsplit; ++z) {
            const size_t idx = ((size_t)z * tokens + tok) * heads + h;
            const float mz = part_ml[idx * 2];
            if (mz != -INFINITY) o += part_o[idx * hd + d] * expf(mz - mmax);
        }
        out[(size_t)tok * out_ld + h * hd + d] = from_float<T>(o * inv);
    }
}


// ---------------------------------------------------------------------------------------
// Tiles of up to 16 query rows in float storage: decoded tokens (the heads of one group are
// the rows) and short portions.  The kernel above gives such a tile to two of its eight warps;
// here all 256 threads work on every chunk of 32 keys:
//   scores   warp w owns rows w and w + 8, lane j key j of the chunk: a dot product over the
//            head with q read as a broadcast and k row j in 16-byte pieces (rows padded by
//            four floats, so the lanes' pieces fall into different banks);
//   softmax  the running maximum and sum of a row live in its warp; the chunk's weights and
//            the row's correction factor go to shared memory;
//   values   thread (row group, four columns of the head) adds the chunk's weighted values to
//            its rows' sums in registers.
// The next chunk's keys and values are copied into the other half of shared memory meanwhile
// (cp.async, 16 bytes at a time, page by page through the block table).
// Same arguments, key ranges, splits and outputs as attn_generic_kernel.  Compiled per head
// size (32, 64, 96, 128, 256), so that every loop over the head unrolls with constant offsets;
// other head sizes take the kernel above.
constexpr int FR = 16;            // rows per tile
constexpr int FK = 32;            // keys per chunk
constexpr int FTHREADS = 256;

__device__ __forceinline__ void copy16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;                     // 0 source bytes: zeros arrive
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

template <int HD>
__global__ void __launch_bounds__(FTHREADS)
attn_rows16_kernel(const AttnParams p) {
    extern __shared__ __align__(16) float fsm[];
    constexpr int hd = HD, kld = HD + 4;
    constexpr int pieces = HD / 4;                                  // 16-byte pieces of a row
    constexpr int row_groups = FTHREADS / pieces;                   // threads side by side along the rows
    constexpr int RPT = (FR + row_groups - 1) / row_groups;         // rows per thread in the values phase
    float* qs = fsm;                                   // [FR][hd], pre-multiplied by the scale
    float* ks = qs + FR * hd;                          // [2][FK][hd + 4]
    float* vs = ks + 2 * FK * kld;                     // [2][FK][hd]
    float* pr = vs + 2 * FK * hd;                      // [FR][FK] weights of the chunk
    float* corr = pr + FR * FK;                        // [FR] correction of the sums so far
    float* lsum = corr + FR;                           // [FR] final sums
    __shared__ long long key_base[3][FK];

    const int kvh = blockIdx.x, tile = blockIdx.y, split = blockIdx.z;
    const int group = p.heads / p.kv_heads;
    const int item = p.tile_item[tile];
    const int row0 = p.tile_row0[tile];
    const int qstart = p.item_qstart[item], qlen = p.item_qlen[item], pos0 = p.item_pos0[item];
    const int nrows = min(FR, qlen * group - row0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* q = (const float*)p.q;
    const float* kp = (const float*)p.k_pages;
    const float* vp = (const float*)p.v_pages;
    const int* bt = p.block_tables + (size_t)item * p.bt_stride;

    for (int e = tid; e < FR * hd; e += FTHREADS) {
        const int r = e / hd, d = e - r * hd;
        float v = 0.f;
        if (r < nrows) {
            const int row = row0 + r;
            const int tok = qstart + row / group, h = kvh * group + row % group;
            v = q[(size_t)tok * p.q_ld + h * hd + d] * p.scale;
        }
        qs[e] = v;
    }

    const int pos_first = pos0 + row0 / group;
    const int pos_last = pos0 + (row0 + nrows - 1) / group;
    int kbegin = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    int kend = pos_last + 1;
    if (p.nsplit > 1) {
        const int span = kend - kbegin;
        int chunk = (span + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + FK - 1) / FK) * FK;
        const int b = kbegin + split * chunk;
        kend = min(kend, b + chunk);
        kbegin = b;
    }
    const int chunks = kend > kbegin ? (kend - kbegin + FK - 1) / FK : 0;

    auto find_rows = [&](int c) {                      // where the keys of chunk c lie in the pages
        if (tid < FK) {
            const int kj = kbegin + c * FK + tid;
            long long base = -1;
            if (c < chunks && kj < kend) {
                const int page = bt[kj / p.page_size];
                if (page >= 0)
                    base = (long long)page * p.page_stride + ((long long)kvh * p.page_size + kj % p.page_size) * hd;
            }
            key_base[c % 3][tid] = base;
        }
    };
    auto fetch = [&](int c) {                          // chunk c's keys and values on their way
        float* kd = ks + (c & 1) * FK * kld;
        float* vd = vs + (c & 1) * FK * hd;
#pragma unroll
        for (int e = tid; e < FK * pieces; e += FTHREADS) {
            const int j = e / pieces, d = (e - j * pieces) * 4;
            const long long base = key_base[c % 3][j];
            copy16(kd + j * kld + d, base >= 0 ? kp + base + d : kp, base >= 0);
            copy16(vd + j * hd + d, base >= 0 ? vp + base + d : vp, base >= 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // rows of this warp in the scores phase, rows and columns of this thread in the values phase
    const int ra = warp, rb = warp + 8;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    const int cg = tid % pieces, rg = tid / pieces;
    const bool has_values = rg < row_groups;
    float4 acc[RPT];
    bool row_on[RPT];                                               // which of this thread's rows exist
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        row_on[i] = has_values && rg + i * row_groups < nrows;
    }

    find_rows(0);
    __syncthreads();                                   // qs and key_base[0] are in place
    if (chunks > 0) fetch(0);
    find_rows(1);
    for (int c = 0; c < chunks; ++c) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                               // chunk c has landed; the last chunk's weights are used up
        if (c + 1 < chunks) fetch(c + 1);
        find_rows(c + 2);
        const float* kc = ks + (c & 1) * FK * kld;
        const float* vc = vs + (c & 1) * FK * hd;
        const int kj = kbegin + c * FK + lane;
        const bool key_ok = kj < kend && key_base[c % 3][lane] >= 0;

        // ---- scores of rows ra and rb against key `lane`
        float s_a = 0.f, s_b = 0.f;
        const bool use_a = ra < nrows, use_b = rb < nrows;
        if (use_a) {
            const float* kr = kc + lane * kld;
            const float* qa = qs + ra * hd;
            const float* qb = qs + rb * hd;
            // four partial sums per row, added at the end: the chain of dependent additions is
            // a quarter as long
            float pa[4] = {0.f, 0.f, 0.f, 0.f}, pb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int d = 0; d < hd; d += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(kr + d);
                const float4 xa = *reinterpret_cast<const float4*>(qa + d);
                pa[0] = fmaf(xa.x, kv.x, pa[0]); pa[1] = fmaf(xa.y, kv.y, pa[1]);
                pa[2] = fmaf(xa.z, kv.z, pa[2]); pa[3] = fmaf(xa.w, kv.w, pa[3]);
                if (use_b) {
                    const float4 xb = *reinterpret_cast<const float4*>(qb + d);
                    pb[0] = fmaf(xb.x, kv.x, pb[0]); pb[1] = fmaf(xb.y, kv.y, pb[1]);
                    pb[2] = fmaf(xb.z, kv.z, pb[2]); pb[3] = fmaf(xb.w, kv.w, pb[3]);
                }
            }
            s_a = (pa[0] + pa[1]) + (pa[2] + pa[3]);
            s_b = (pb[0] + pb[1]) + (pb[2] + pb[3]);
        }
        // ---- running softmax of the two rows; weights and corrections to shared memory
        auto update = [&](int r, bool used, float s, float& m, float& l) {
            float pj = 0.f, factor = 1.f;
            if (used) {
                const int pos = pos0 + (row0 + r) / group;
                const bool seen = key_ok && kj <= pos && (p.window <= 0 || kj > pos - p.window);
                s = seen ? s : -INFINITY;
                const float m_new = fmaxf(m, warp_max(s));
                if (m_new != -INFINITY) {
                    factor = expf(m - m_new);             // m = -inf gives 0
                    pj = seen ? expf(s - m_new) : 0.f;
                    l = l * factor + warp_sum(pj);
                    m = m_new;
                }
            }
            pr[r * FK + lane] = pj;
            if (lane == 0) corr[r] = factor;
        };
        update(ra, use_a, s_a, m_a, l_a);
        update(rb, use_b, s_b, m_b, l_b);
        __syncthreads();
        // ---- weighted values
        if (row_on[0]) {                               // a thread's first row exists if any of its rows does
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                if (row_on[i]) {
                    const float f = corr[rg + i * row_groups];
                    acc[i].x *= f; acc[i].y *= f; acc[i].z *= f; acc[i].w *= f;
                }
            }
            const float* vcol = vc + cg * 4;
#pragma unroll 8
            for (int j = 0; j < FK; ++j) {
                const float4 vv = *reinterpret_cast<const float4*>(vcol + j * hd);
#pragma unroll
                for (int i = 0; i < RPT; ++i) {
                    if (row_on[i]) {
                        const float w = pr[(rg + i * row_groups) * FK + j];
                        acc[i].x = fmaf(w, vv.x, acc[i].x); acc[i].y = fmaf(w, vv.y, acc[i].y);
                        acc[i].z = fmaf(w, vv.z, acc[i].z); acc[i].w = fmaf(w, vv.w, acc[i].w);
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // ---- results: the sums of a row are with its warp, its weighted values with other threads
    if (lane == 0) {
        if (ra < nrows) {
            lsum[ra] = l_a;
            if (p.nsplit > 1) {
                const int row = row0 + ra;
                const size_t idx = ((size_t)split * p.tokens + qstart + row / group) * p.heads + kvh * group + row % group;
                p.part_ml[idx * 2] = m_a; p.part_ml[idx * 2 + 1] = l_a;
            }
        }
        if (rb < nrows) {
            lsum[rb] = l_b;
            if (p.nsplit > 1) {
                const int row = row0 + rb;
                const size_t idx = ((size_t)split * p.tokens + qstart + row / group) * p.heads + kvh * group + row % group;
                p.part_ml[idx * 2] = m_b; p.part_ml[idx * 2 + 1] = l_b;
            }
        }
    }
    __syncthreads();
    if (has_values) {
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            const int r = rg + i * row_groups;
            if (!row_on[i]) continue;
            const int row = row0 + r;
            const int tok = qstart + row / group, h = kvh * group + row % group;
            if (p.nsplit == 1) {
                const float l = lsum[r];
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                float* o = (float*)p.out + (size_t)tok * p.out_ld + h * hd + cg * 4;
                o[0] = acc[i].x * inv; o[1] = acc[i].y * inv; o[2] = acc[i].z * inv; o[3] = acc[i].w * inv;
            } else {
                const size_t idx = ((size_t)split * p.tokens + tok) * p.heads + h;
                float* o = p.part_o + idx * hd + cg * 4;
                o[0] = acc[i].x; o[1] = acc[i].y; o[2] = acc[i].z; o[3] = acc[i].w;
            }
        }
    }
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_attn_generic_rows() { return ROWS; }
int fsie_attn_rows16_rows() { return FR; }
// head sizes the kernel for tiles of up to 16 rows is compiled for
int fsie_attn_rows16_takes(int head_dim) {
    return head_dim == 32 || head_dim == 64 || head_dim == 96 || head_dim == 128 || head_dim == 256;
}

// Launch over `tiles` row tiles.  With nsplit > 1 the caller provides part_o
// [nsplit, tokens, heads, head_dim] and part_ml [nsplit, tokens, heads, 2] in float.
// rows16: the tiles hold up to 16 rows and take attn_rows16_kernel (float storage, head sizes in
// steps of 4); else up to 32 rows and attn_generic_kernel.  merge: the partial results of all
// tokens are merged after this launch (a step whose tiles go out in several launches asks for
// it with the last one only).
int fsie_attn_tiles(const void* q, int q_ld, const void* k_pages, const void* v_pages,
                    long long page_stride, int page_size, const int* block_tables, int bt_stride,
                    const int* tile_item, const int* tile_row0, int tiles,
                    const int* item_qstart, const int* item_qlen, const int* item_pos0,
                    void* out, int out_ld, float* part_o, float* part_ml, int tokens, int heads,
                    int kv_heads, int head_dim, int window, int nsplit, float scale, int dtype,
                    int rows16, int merge, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (tiles > 65535) return ERR_UNSUPPORTED;          // tiles are the grid's y dimension
    if (head_dim <= 0 || head_dim > 32 * MAX_DPL || kv_heads <= 0 || heads % kv_heads != 0 ||
        nsplit < 1 || page_size <= 0 || tiles < 0)
        return ERR_BAD_ARGUMENT;
    if (nsplit > 1 && (!part_o || !part_ml)) return ERR_BAD_ARGUMENT;
    if (rows16 && (dtype != DTYPE_F32 || !fsie_attn_rows16_takes(head_dim) || page_stride % 4 != 0 ||
                   ((((size_t)k_pages) | ((size_t)v_pages)) & 15) != 0))
        return ERR_UNSUPPORTED;
    AttnParams p;
    p.q = q; p.q_ld = q_ld; p.k_pages = k_pages; p.v_pages = v_pages;
    p.page_stride = page_stride; p.page_size = page_size;
    p.block_tables = block_tables; p.bt_stride = bt_stride;
    p.tile_item = tile_item; p.tile_row0 = tile_row0;
    p.item_qstart = item_qstart; p.item_qlen = item_qlen; p.item_pos0 = item_pos0;
    p.out = out; p.out_ld = out_ld; p.part_o = part_o; p.part_ml = part_ml;
    p.tokens = tokens; p.heads = heads; p.kv_heads = kv_heads; p.head_dim = head_dim;
    p.window = window; p.nsplit = nsplit; p.scale = scale;
    int rc = 0;
    if (tiles > 0) {
        dim3 grid(kv_heads, tiles, nsplit);
        if (rows16) {
            const size_t smem = sizeof(float) * ((size_t)FR * head_dim + 2 * (size_t)FK * (head_dim + 4) +
                                                 2 * (size_t)FK * head_dim + (size_t)FR * FK + 2 * FR);
#define FSIE_ROWS16(HDV)                                                                                        \
    case HDV:                                                                                                   \
        cudaFuncSetAttribute(attn_rows16_kernel<HDV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        attn_rows16_kernel<HDV><<<grid, FTHREADS, smem, stream>>>(p);                                           \
        break;
            switch (head_dim) {
                FSIE_ROWS16(32) FSIE_ROWS16(64) FSIE_ROWS16(96) FSIE_ROWS16(128) FSIE_ROWS16(256)
                default: return ERR_UNSUPPORTED;
            }
#undef FSIE_ROWS16
        } else {
            const size_t smem = sizeof(float) * ((size_t)ROWS * head_dim + (size_t)KT * (head_dim + 1) +
                                                 (size_t)KT * head_dim);
            if (dtype == DTYPE_F32) {
                cudaFuncSetAttribute(attn_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                attn_generic_kernel<float><<<grid, WARPS * 32, smem, stream>>>(p);
            } else {
                cudaFuncSetAttribute(attn_generic_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                attn_generic_kernel<bf16><<<grid, WARPS * 32, smem, stream>>>(p);
            }
        }
        rc = FSIE_LAUNCH_CHECK();
    }
    if (rc != 0 || nsplit == 1 || !merge) return rc;
    dim3 cgrid(tokens, heads);
    const int threads = head_dim >= 128 ? 128 : (head_dim >= 64 ? 64 : 32);
    if (dtype == DTYPE_F32)
        attn_combine_kernel<float><<<cgrid, threads, 0, stream>>>(part_o, part_ml, (float*)out, out_ld, tokens, heads, head_dim, nsplit);
    else
        attn_combine_kernel<bf16><<<cgrid, threads, 0, stream>>>(part_o, part_ml, (bf16*)out, out_ld, tokens, heads, head_dim, nsplit);
    return FSIE_LAUNCH_CHECK();
}

// The launch as callers outside the engine know it: tiles of up to 32 rows, merged at once.
int fsie_attn_generic(const void* q, int q_ld, const void* k_pages, const void* v_pages,
                      long long page_stride, int page_size, const int* block_tables, int bt_stride,
                      const int* tile_item, const int* tile_row0, int tiles,
                      const int* item_qstart, const int* item_qlen, const int* item_pos0,
                      void* out, int out_ld, float* part_o, float* part_ml, int tokens, int heads,
                      int kv_heads, int head_dim, int window, int nsplit, float scale, int dtype,
                      cudaStream_t stream) {
    if (tiles <= 0 || tokens <= 0) return 0;
    return fsie_attn_tiles(q, q_ld, k_pages, v_pages, page_stride, page_size, block_tables, bt_stride,
                           tile_item, tile_row0, tiles, item_qstart, item_qlen, item_pos0, out, out_ld,
                           part_o, part_ml, tokens, heads, kv_heads, head_dim, window, nsplit, scale,
                           dtype, 0, 1, stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// The same launch for callers that cannot allocate: the split results live in a fixed
// array of this library instead of caller-provided buffers (see attention_static_scratch.h).
#include "attention_static_scratch.h"

namespace fsie {

static __device__ __align__(256) float static_scratch[FSIE_STATIC_SCRATCH_FLOATS];

// Device address of static_scratch per device ordinal, looked up once per device.  In host
// code the array's name is only a handle for the runtime, not an address a kernel can use.
constexpr int MAX_DEVICES = 64;
static float* scratch_address[MAX_DEVICES] = {};

static int static_scratch_for_current_device(float** address) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES)
        return FSIE_ERR_SCRATCH_SETUP;
    if (scratch_address[device] == nullptr) {
        float* found = nullptr;
        if (cudaGetSymbolAddress((void**)&found, static_scratch) != cudaSuccess || !found)
            return FSIE_ERR_SCRATCH_SETUP;
        scratch_address[device] = found;
    }
    *address = scratch_address[device];
    return 0;
}

}  // namespace fsie

extern "C" {

long long fsie_attn_static_scratch_floats(int tokens, int heads, int head_dim, int nsplit) {
    if (nsplit <= 1) return 0;
    if (tokens < 0 || heads < 0 || head_dim < 0) return -1;
    // multiplied factor by factor and cut off as soon as the limit is passed, so that four
    // large ints cannot wrap around 64 bits and slip under the check
    const long long limit = (long long)FSIE_STATIC_SCRATCH_FLOATS;
    const long long factors[4] = {nsplit, tokens, heads, (long long)head_dim + 2};
    long long need = 1;
    for (long long f : factors) {
        if (f > limit) return limit + 1;
        need *= f;                         // need <= limit and f <= limit: below 2^40
        if (need > limit) return limit + 1;
    }
    return need;
}

const char* fsie_attn_static_scratch_error(int code) {
    switch (code) {
        case 0: return "ok";
        case FSIE_ERR_SCRATCH_TOO_SMALL:
            return "the launch needs more split scratch than the library's fixed array holds "
                   "(nsplit * tokens * heads * (head_dim + 2) floats > FSIE_STATIC_SCRATCH_FLOATS); "
                   "use fewer splits or fewer tokens per call, or fsie_attn_generic with your own buffers";
        case FSIE_ERR_SCRATCH_SETUP:
            return "the device address of the library's scratch array could not be looked up "
                   "on the current device";
        case fsie::ERR_BAD_ARGUMENT: return "an argument was refused by the launcher";
        default: return "CUDA error (the code is a cudaError_t)";
    }
}

int fsie_attn_generic_static_scratch(
    const void* q, int q_ld, const void* k_pages, const void* v_pages, long long page_stride,
    int page_size, const int* block_tables, int bt_stride, const int* tile_item,
    const int* tile_row0, int tiles, const int* item_qstart, const int* item_qlen,
    const int* item_pos0, void* out, int out_ld, int tokens, int heads, int kv_heads,
    int head_dim, int window, int nsplit, float scale, int dtype, cudaStream_t stream) {
    if (tokens < 0 || heads <= 0 || head_dim <= 0 || nsplit < 1) return fsie::ERR_BAD_ARGUMENT;
    const long long need = fsie_attn_static_scratch_floats(tokens, heads, head_dim, nsplit);
    if (need < 0) return fsie::ERR_BAD_ARGUMENT;
    if (need > (long long)FSIE_STATIC_SCRATCH_FLOATS) return FSIE_ERR_SCRATCH_TOO_SMALL;
    float* scratch = nullptr;
    const int rc = fsie::static_scratch_for_current_device(&scratch);
    if (rc != 0) return rc;
    // [nsplit, tokens, heads, head_dim] partial sums, then [nsplit, tokens, heads, 2] (max, sum)
    float* part_o = scratch;
    float* part_ml = scratch + (long long)nsplit * tokens * heads * head_dim;
    return fsie_attn_generic(q, q_ld, k_pages, v_pages, page_stride, page_size, block_tables,
                             bt_stride, tile_item, tile_row0, tiles, item_qstart, item_qlen,
                             item_pos0, out, out_ld, part_o, part_ml, tokens, heads, kv_heads,
                             head_dim, window, nsplit, scale, dtype, stream);
}

}  // extern "C"
