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
    const int row = blockIdx.y, part = blockIdx.x;
    const float* src = logits + (size_t)row * vocab;
    const int seg = (vocab + parts - 1) / parts;
    const int begin = part * seg, end = min(vocab, begin + seg);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll 4
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = src[i];
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
        part_v[(size_t)row * parts + part] = bv;
        part_i[(size_t)row * parts + part] = bi;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                    int parts, int* __restrict__ out) {
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
    fsie::argmax_partial_kernel<<<dim3(parts, rows), 256, 0, stream>>>(logits, vocab, parts, part_v, part_i);
    fsie::argmax_final_kernel<<<rows, 32, 0, stream>>>(part_v, part_i, parts, out);
    return FSIE_LAUNCH_CHECK();
}

// Rows with temperature <= 0 get -1 (use fsie_argmax for them).
int fsie_sample(const float* logits, int rows, int vocab, const float* temperature,
                const int* top_k, const float* top_p, const float* uniform, int* out,
                cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return fsie::ERR_BAD_ARGUMENT;
    fsie::sample_kernel<<<rows, fsie::SAMPLE_THREADS, 0, stream>>>(logits, vocab, temperature, top_k,
                                                                  top_p, uniform, out);
    return FSIE_LAUNCH_CHECK();
}

}  // extern "C"
