// Next-token choice on the device: argmax, and temperature -> top-k -> top-p -> draw.
//
// Meaning as the reference sampler (src/sampler/sampler.cpp:25-88): with
// temperature <= 0 the first largest logit wins; otherwise the tokens are taken in
// order of descending logit, cut to the top_k first (0 = all), given probabilities
// softmax(logit / temperature), cut to the shortest prefix whose mass reaches top_p
// (>= 1 = all), and the token is found by walking that prefix until the running mass
// reaches u * (mass of the prefix).  The reference sorts the whole vocabulary on the
// host; here nothing is sorted.  "The running mass over tokens in descending order
// reaches a target" is answered by a search over the 32 bits of an order-preserving
// integer key of the logit: each of the 32 rounds measures the mass (or the count) of
// all tokens whose key is at least a candidate, with a block reduction in a fixed
// order.  Tokens with equal logits are ordered by ascending index.  The uniform number
// u in [0,1) comes from the host, one per row, so a request's draws do not depend on
// what else is in the batch.
#include "common.cuh"
#include <cooperative_groups.h>
#include <math.h>

namespace fsie {

constexpr int SAMPLE_THREADS = 1024;

// float -> unsigned key with the same order (NaN sorts below everything as key 0)
__device__ __forceinline__ unsigned order_key(float v) {
    if (v != v) return 0u;
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned block_count(unsigned v, unsigned* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    unsigned total = 0;
    for (int w = 0; w < warps; ++w) total += scratch[w];
    return total;
}

// One block per row: the index of the largest logit, ties to the smallest index
// (src/cuda/device.cu:232-266 has the same tie rule).
__global__ void argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int warps = (blockDim.x + 31) >> 5;
        for (int w = 1; w < warps; ++w)
            if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
        out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// The same in two stages for wide vocabularies: `parts` blocks per row each reduce a
// segment to (value, index), one warp per row picks among them.
__global__ void argmax_partial_kernel(const float* __restrict__ logits, int vocab, int parts,
                                      float* __restrict__ part_v, int* __restrict__ part_i) {
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    grid_dependency_wait();
    grid_dependents_go();
    const int row = blockIdx.y, part = blockIdx.x;
    const float* src = logits + (size_t)row * vocab;
    const int seg = (((vocab + parts - 1) / parts) + 3) & ~3;
    const int begin = min(vocab, part * seg), end = min(vocab, begin + seg);
    // a thread meets its indices in rising order: "greater" alone keeps the first of equals
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        // 16 bytes per load, two loads in flight
        int i = begin + 4 * threadIdx.x;
        const int step = 4 * blockDim.x;
        for (; i + step + 3 < end; i += 2 * step) {
            const float4 a = *reinterpret_cast<const float4*>(src + i);
            const float4 b = *reinterpret_cast<const float4*>(src + i + step);
            if (a.x > bv) { bv = a.x; bi = i; }
            if (a.y > bv) { bv = a.y; bi = i + 1; }
            if (a.z > bv) { bv = a.z; bi = i + 2; }
            if (a.w > bv) { bv = a.w; bi = i + 3; }
            if (b.x > bv) { bv = b.x; bi = i + step; }
            if (b.y > bv) { bv = b.y; bi = i + step + 1; }
            if (b.z > bv) { bv = b.z; bi = i + step + 2; }
            if (b.w > bv) { bv = b.w; bi = i + step + 3; }
        }
        for (; i + 3 < end; i += step) {
            const float4 a = *reinterpret_cast<const float4*>(src + i);
            if (a.x > bv) { bv = a.x; bi = i; }
            if (a.y > bv) { bv = a.y; bi = i + 1; }
            if (a.z > bv) { bv = a.z; bi = i + 2; }
            if (a.w > bv) { bv = a.w; bi = i + 3; }
        }
    } else {
#pragma unroll 4
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
            const float v = src[i];
            if (v > bv) { bv = v; bi = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int warps = (blockDim.x + 31) >> 5;
        for (int w = 1; w < warps; ++w)
            if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
        part_v[(size_t)row * parts + part] = bv;
        part_i[(size_t)row * parts + part] = bi;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                    int parts, int* __restrict__ out) {
    grid_dependency_wait();
    grid_dependents_go();
    const int row = blockIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int p = threadIdx.x; p < parts; p += 32) {
        const float v = part_v[(size_t)row * parts + p];
        const int i = part_i[(size_t)row * parts + p];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (threadIdx.x == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

struct RowView {
    const float* row; int vocab; float inv_temp; float maxl;
    unsigned kept_key;     // top-k boundary: every key above it is kept ...
    unsigned kept_ties;    // ... and of the tokens at it, the first kept_ties by index
};

__device__ __forceinline__ float weight_of(const RowView& r, int i) {
    return expf((r.row[i] - r.maxl) * r.inv_temp);
}

struct Located { unsigned key; float above; float w; unsigned count; };

// Walk the kept tokens in descending order until the running weight reaches `target`:
// returns the key K at which that happens (the largest K with weight(key >= K) >= target),
// the weight strictly above K, the weight of one token at K and how many kept tokens sit at K.
__device__ Located locate(const RowView& r, float target, float* scratch, unsigned* uscratch) {
    unsigned prefix = 0;
    for (int bit = 31; bit >= 0; --bit) {
        const unsigned cand = prefix | (1u << bit);
        bool reached = cand <= r.kept_key;        // at or below the boundary: the whole kept set
        if (!reached && target != INFINITY) {
            float mass = 0.f;
            for (int i = threadIdx.x; i < r.vocab; i += blockDim.x)
                if (order_key(r.row[i]) >= cand) mass += weight_of(r, i);
            const float total = block_sum(mass, scratch);
            reached = total >= target && total > 0.f;   // target 0 stops at the first token
        }
        if (reached) prefix = cand;
    }
    Located out;
    out.key = prefix;
    float above = 0.f, w = 0.f;
    unsigned count = 0;
    for (int i = threadIdx.x; i < r.vocab; i += blockDim.x) {
        const unsigned key = order_key(r.row[i]);
        if (key > prefix) above += weight_of(r, i);
        else if (key == prefix) { count += 1; w = weight_of(r, i); }
    }
    out.above = block_sum(above, scratch);
    out.w = block_max(w, scratch);
    out.count = block_count(count, uscratch);
    if (prefix == r.kept_key && r.kept_ties < out.count) out.count = r.kept_ties;
    return out;
}

// how many tokens at the located key are needed for the running weight to reach target
__device__ __forceinline__ unsigned ties_needed(const Located& at, float target) {
    if (at.count <= 1 || !(at.w > 0.f)) return 1;
    const float n = ceilf((target - at.above) / at.w);
    if (!(n >= 1.f)) return 1;
    return n >= (float)at.count ? at.count : (unsigned)n;
}

// index of the n-th (1-based, by ascending index) token whose key equals `key`
__device__ int nth_with_key(const RowView& r, unsigned key, unsigned n, unsigned* counts,
                            int* result) {
    const int per = (r.vocab + blockDim.x - 1) / blockDim.x;   // contiguous chunk per thread
    const int begin = threadIdx.x * per, end = min(r.vocab, begin + per);
    unsigned mine = 0;
    for (int i = begin; i < end; ++i) mine += order_key(r.row[i]) == key;
    __syncthreads();
    counts[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned run = 0;
        int found = -1;
        for (int t = 0; t < (int)blockDim.x && found < 0; ++t) {
            if (run + counts[t] >= n) {
                const int b = t * per, e = min(r.vocab, b + per);
                for (int i = b; i < e; ++i)
                    if (order_key(r.row[i]) == key && ++run == n) { found = i; break; }
            } else {
                run += counts[t];
            }
        }
        *result = found;
    }
    __syncthreads();
    return *result;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ float scratch[32];
    __shared__ unsigned uscratch[32];
    __shared__ unsigned counts[SAMPLE_THREADS];
    __shared__ int found;
    const int rix = blockIdx.x;
    RowView r;
    r.row = logits + (size_t)rix * vocab;
    r.vocab = vocab;
    const float temp = temperature[rix];
    if (!(temp > 0.f)) {       // greedy rows are served by argmax_kernel; keep a defined value
        if (threadIdx.x == 0) out[rix] = -1;
        return;
    }
    r.inv_temp = 1.0f / temp;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, r.row[i]);
    r.maxl = block_max(mx, scratch);

    // ---- top-k: the key of the k-th largest logit and how many of its ties are kept
    r.kept_key = 0;
    r.kept_ties = 0xffffffffu;
    const int k = top_k[rix];
    if (k > 0 && k < vocab) {
        unsigned prefix = 0;   // largest K with count(key >= K) >= k
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = prefix | (1u << bit);
            unsigned c = 0;
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += order_key(r.row[i]) >= cand;
            if (block_count(c, uscratch) >= (unsigned)k) prefix = cand;
        }
        unsigned above = 0;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) above += order_key(r.row[i]) > prefix;
        r.kept_key = prefix;
        r.kept_ties = (unsigned)k - block_count(above, uscratch);
    }

    // ---- weight of the kept set (a target no finite weight reaches lands on the boundary)
    const Located whole = locate(r, INFINITY, scratch, uscratch);
    const float total = whole.above + (float)whole.count * whole.w;

    // ---- top-p: weight of the shortest descending prefix that reaches top_p * total
    float nucleus = total;
    const float pp = top_p[rix];
    if (pp < 1.0f) {
        const float target = pp * total;
        const Located at = locate(r, target, scratch, uscratch);
        nucleus = at.above + (float)ties_needed(at, target) * at.w;
    }

    // ---- draw: the first token whose running weight reaches u * nucleus
    const float target = uniform[rix] * nucleus;
    const Located at = locate(r, target, scratch, uscratch);
    const int choice = nth_with_key(r, at.key, ties_needed(at, target), counts, &found);
    if (threadIdx.x == 0) out[rix] = choice < 0 ? 0 : choice;
}

// ------------------------------------------------------------------ cluster version
// The same choice with a cluster of CLUSTER blocks per row (thread-block clusters,
// distributed shared memory).  Each block keeps its slice of the row in shared memory as
// (order key, weight) pairs, computed once, so the 32 rounds of a search read shared
// memory only; the blocks' partial sums meet through distributed shared memory, summed in
// rank order (the same bits on every run).  Rows then take microseconds per round instead
// of a pass over global memory by a single block.
namespace cg = cooperative_groups;
constexpr int CLUSTER = 8;

struct ClusterRow {
    const unsigned* keys; const float* w; int count;    // this block's slice
    int first;                                           // index of its first element in the row
    unsigned kept_key, kept_ties;
    float* slots;                                        // [2][4] exchange area of this block
    int parity;
};

// sum over the cluster in rank order; every block gets the same bits
__device__ float cluster_sum(cg::cluster_group& cluster, ClusterRow& r, float v, float* scratch) {
    v = block_sum(v, scratch);
    float* mine = r.slots + r.parity * 4;
    if (threadIdx.x == 0) mine[0] = v;
    cluster.sync();
    float total = 0.f;
    for (int rank = 0; rank < CLUSTER; ++rank)
        total += (cluster.map_shared_rank(r.slots, rank) + r.parity * 4)[0];
    r.parity ^= 1;
    return total;
}

// three sums at once (one block reduction, one exchange); `wide` holds 96 floats
__device__ void cluster_sum3(cg::cluster_group& cluster, ClusterRow& r, float (&v)[3], float* wide) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int j = 0; j < 3; ++j) v[j] = warp_sum(v[j]);
    __syncthreads();
    if (lane == 0) { wide[warp * 3] = v[0]; wide[warp * 3 + 1] = v[1]; wide[warp * 3 + 2] = v[2]; }
    __syncthreads();
    float* mine = r.slots + r.parity * 4;
    if (threadIdx.x < 3) {
        float total = 0.f;
        for (int w = 0; w < warps; ++w) total += wide[w * 3 + threadIdx.x];
        mine[threadIdx.x] = total;
    }
    cluster.sync();
    v[0] = v[1] = v[2] = 0.f;
    for (int rank = 0; rank < CLUSTER; ++rank) {
        const float* theirs = cluster.map_shared_rank(r.slots, rank) + r.parity * 4;
        v[0] += theirs[0]; v[1] += theirs[1]; v[2] += theirs[2];
    }
    r.parity ^= 1;
}

struct Found { unsigned key; float above; float w; float count; };

// as locate() above, over the cluster's shared-memory copy of the row
__device__ Found cluster_locate(cg::cluster_group& cluster, ClusterRow& r, float target, float* scratch,
                               float* wide) {
    // two key bits per round: the weights at or above the three candidates prefix + {1,2,3} * 2^lo
    unsigned prefix = 0;
    for (int lo = 30; lo >= 0; lo -= 2) {
        const unsigned c1 = prefix | (1u << lo), c2 = prefix | (2u << lo), c3 = prefix | (3u << lo);
        float m[3] = {0.f, 0.f, 0.f};
        if (c3 > r.kept_key && target != INFINITY) {
            for (int i = threadIdx.x; i < r.count; i += blockDim.x) {
                const unsigned key = r.keys[i];
                const float wi = r.w[i];
                if (key >= c1) m[0] += wi;
                if (key >= c2) m[1] += wi;
                if (key >= c3) m[2] += wi;
            }
            cluster_sum3(cluster, r, m, wide);
        }
        const bool inf = target == INFINITY;
        const bool r1 = c1 <= r.kept_key || (!inf && m[0] >= target && m[0] > 0.f);
        const bool r2 = c2 <= r.kept_key || (!inf && m[1] >= target && m[1] > 0.f);
        const bool r3 = c3 <= r.kept_key || (!inf && m[2] >= target && m[2] > 0.f);
        if (r3) prefix = c3; else if (r2) prefix = c2; else if (r1) prefix = c1;
    }
    float v[3] = {0.f, 0.f, 0.f};      // weight above, tokens at the key, weight of one of them
    float w_at = 0.f;
    for (int i = threadIdx.x; i < r.count; i += blockDim.x) {
        const unsigned key = r.keys[i];
        if (key > prefix) v[0] += r.w[i];
        else if (key == prefix) { v[1] += 1.f; w_at = r.w[i]; }
    }
    v[2] = block_max(w_at, scratch);   // equal keys have equal weights: max picks it
    // max over the cluster through the same exchange: send it as a sum of one-hot parts
    float* mine = r.slots + r.parity * 4;
    v[0] = block_sum(v[0], scratch);
    v[1] = block_sum(v[1], scratch);
    if (threadIdx.x == 0) { mine[0] = v[0]; mine[1] = v[1]; mine[2] = v[2]; }
    cluster.sync();
    Found out;
    out.key = prefix; out.above = 0.f; out.count = 0.f; out.w = 0.f;
    for (int rank = 0; rank < CLUSTER; ++rank) {
        const float* theirs = cluster.map_shared_rank(r.slots, rank) + r.parity * 4;
        out.above += theirs[0]; out.count += theirs[1]; out.w = fmaxf(out.w, theirs[2]);
    }
    r.parity ^= 1;
    if (prefix == r.kept_key && (float)r.kept_ties < out.count) out.count = (float)r.kept_ties;
    return out;
}

__device__ __forceinline__ unsigned cluster_ties_needed(const Found& at, float target) {
    if (at.count <= 1.f || !(at.w > 0.f)) return 1;
    const float n = ceilf((target - at.above) / at.w);
    if (!(n >= 1.f)) return 1;
    return n >= at.count ? (unsigned)at.count : (unsigned)n;
}

__global__ void __cluster_dims__(CLUSTER, 1, 1) __launch_bounds__(SAMPLE_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, int vocab, int slice,
                      const float* __restrict__ temperature, const int* __restrict__ top_k,
                      const float* __restrict__ top_p, const float* __restrict__ uniform,
                      int* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char sample_smem[];
    __shared__ float scratch[32];
    __shared__ float wide[96];
    __shared__ float slots[2 * 4];
    __shared__ unsigned counts[SAMPLE_THREADS];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int rix = blockIdx.y;
    const float temp = temperature[rix];
    if (!(temp > 0.f)) {                         // uniform over the cluster: no sync is skipped
        if (rank == 0 && threadIdx.x == 0) out[rix] = -1;
        return;
    }
    unsigned* keys = reinterpret_cast<unsigned*>(sample_smem);
    float* w = reinterpret_cast<float*>(sample_smem) + slice;
    ClusterRow r;
    r.first = rank * slice;
    r.count = max(0, min(slice, vocab - r.first));
    r.keys = keys; r.w = w; r.slots = slots; r.parity = 0;
    const float* row = logits + (size_t)rix * vocab + r.first;
    const float inv_temp = 1.0f / temp;

    // ---- the row's maximum, then this block's (key, weight) pairs
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < r.count; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = block_max(mx, scratch);
    if (threadIdx.x == 0) slots[0] = mx;
    cluster.sync();
    float maxl = -INFINITY;
    for (int q = 0; q < CLUSTER; ++q) maxl = fmaxf(maxl, cluster.map_shared_rank(slots, q)[0]);
    cluster.sync();                              // everyone has read slot 0 before it is reused
    for (int i = threadIdx.x; i < r.count; i += blockDim.x) {
        const float v = row[i];
        keys[i] = order_key(v);
        w[i] = expf((v - maxl) * inv_temp);
    }
    __syncthreads();

    // ---- top-k: key of the k-th largest logit, and how many of its ties are kept
    r.kept_key = 0; r.kept_ties = 0xffffffffu;
    const int k = top_k[rix];
    if (k > 0 && k < vocab) {
        unsigned prefix = 0;                             // largest key with count(key >= it) >= k
        for (int lo = 30; lo >= 0; lo -= 2) {
            const unsigned c1 = prefix | (1u << lo), c2 = prefix | (2u << lo), c3 = prefix | (3u << lo);
            float c[3] = {0.f, 0.f, 0.f};                // counts up to 2^24 are exact in float
            for (int i = threadIdx.x; i < r.count; i += blockDim.x) {
                const unsigned key = keys[i];
                c[0] += key >= c1 ? 1.f : 0.f; c[1] += key >= c2 ? 1.f : 0.f; c[2] += key >= c3 ? 1.f : 0.f;
            }
            cluster_sum3(cluster, r, c, wide);
            if (c[2] >= (float)k) prefix = c3; else if (c[1] >= (float)k) prefix = c2;
            else if (c[0] >= (float)k) prefix = c1;
        }
        float above = 0.f;
        for (int i = threadIdx.x; i < r.count; i += blockDim.x) above += keys[i] > prefix ? 1.f : 0.f;
        above = cluster_sum(cluster, r, above, scratch);
        r.kept_key = prefix;
        r.kept_ties = (unsigned)k - (unsigned)above;
    }
    const Found whole = cluster_locate(cluster, r, INFINITY, scratch, wide);
    const float total = whole.above + whole.count * whole.w;
    float nucleus = total;
    const float pp = top_p[rix];
    if (pp < 1.0f) {
        const float target = pp * total;
        const Found at = cluster_locate(cluster, r, target, scratch, wide);
        nucleus = at.above + (float)cluster_ties_needed(at, target) * at.w;
    }
    const float target = uniform[rix] * nucleus;
    const Found at = cluster_locate(cluster, r, target, scratch, wide);
    unsigned n = cluster_ties_needed(at, target);

    // ---- the n-th token (by ascending index) whose key equals at.key: which block holds it?
    float mine[3] = {0.f, 0.f, 0.f};
    for (int i = threadIdx.x; i < r.count; i += blockDim.x) mine[0] += keys[i] == at.key ? 1.f : 0.f;
    mine[0] = block_sum(mine[0], scratch);
    float* slot = r.slots + r.parity * 4;
    if (threadIdx.x == 0) slot[0] = mine[0];
    cluster.sync();
    unsigned before = 0, here = 0, all = 0;
    for (int q = 0; q < CLUSTER; ++q) {
        const unsigned c = (unsigned)(cluster.map_shared_rank(r.slots, q) + r.parity * 4)[0];
        if (q < rank) before += c;
        if (q == rank) here = c;
        all += c;
    }
    if (n > all) n = all;
    if (all == 0 && rank == 0 && threadIdx.x == 0) out[rix] = 0;
    if (n > before && n <= before + here) {       // this block owns the answer
        const unsigned local = n - before;
        const int per = (r.count + blockDim.x - 1) / blockDim.x;
        const int begin = threadIdx.x * per, end = min(r.count, begin + per);
        unsigned cnt = 0;
        for (int i = begin; i < end; ++i) cnt += keys[i] == at.key;
        counts[threadIdx.x] = cnt;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned run = 0;
            int found = -1;
            for (int t = 0; t < (int)blockDim.x && found < 0; ++t) {
                if (run + counts[t] >= local) {
                    const int b = t * per, e = min(r.count, b + per);
                    for (int i = b; i < e; ++i)
                        if (keys[i] == at.key && ++run == local) { found = i; break; }
                } else {
                    run += counts[t];
                }
            }
            out[rix] = found < 0 ? 0 : r.first + found;
        }
    }
    cluster.sync();                               // no block leaves while its slots may be read
}

}  // namespace fsie

extern "C" {

int fsie_argmax(const float* logits, int rows, int vocab, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return fsie::ERR_BAD_ARGUMENT;
    fsie::argmax_kernel<<<rows, 1024, 0, stream>>>(logits, vocab, out);
    return FSIE_LAUNCH_CHECK();
}

// Two-stage argmax; `scratch` holds rows * parts floats followed by rows * parts ints.
int fsie_argmax_staged(const float* logits, int rows, int vocab, int* out, void* scratch, int parts,
                       cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || parts <= 0 || !scratch) return fsie::ERR_BAD_ARGUMENT;
    float* part_v = (float*)scratch;
    int* part_i = (int*)scratch + (size_t)rows * parts;
    int rc = fsie::launch_dependent(fsie::argmax_partial_kernel, dim3(parts, rows), dim3(256), 0, stream, logits, vocab, parts, part_v, part_i);
    if (rc != 0) return rc;
    return fsie::launch_dependent(fsie::argmax_final_kernel, dim3(rows), dim3(32), 0, stream, (const float*)part_v, (const int*)part_i, parts, out);
    return FSIE_LAUNCH_CHECK();
}

// Rows with temperature <= 0 get -1 (use fsie_argmax for them).
int fsie_sample(const float* logits, int rows, int vocab, const float* temperature,
                const int* top_k, const float* top_p, const float* uniform, int* out,
                cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return fsie::ERR_BAD_ARGUMENT;
    // a cluster of 8 blocks per row while a slice of the row fits in shared memory
    const int slice = ((vocab + fsie::CLUSTER - 1) / fsie::CLUSTER + 3) / 4 * 4;
    const size_t smem = (size_t)slice * 8;
    if (vocab >= 4096 && smem <= 200 * 1024 && rows <= 65535) {
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(fsie::sample_cluster_kernel,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
        fsie::sample_cluster_kernel<<<dim3(fsie::CLUSTER, rows), fsie::SAMPLE_THREADS, smem, stream>>>(
            logits, vocab, slice, temperature, top_k, top_p, uniform, out);
        return FSIE_LAUNCH_CHECK();
    }
    fsie::sample_kernel<<<rows, fsie::SAMPLE_THREADS, 0, stream>>>(logits, vocab, temperature, top_k,
                                                                  top_p, uniform, out);
    return FSIE_LAUNCH_CHECK();
}

}  // extern "C"
