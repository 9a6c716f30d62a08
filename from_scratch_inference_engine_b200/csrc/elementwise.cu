// Row-wise and element-wise kernels of the decoder step: embedding gather, fused
// residual add + RMSNorm, rotary position encoding fused with the paged cache write,
// and SwiGLU.  Each is templated on the storage type (float for the 32-bit path,
// bfloat16 for serving); every reduction and the residual stream are 32-bit.
#include "common.cuh"

namespace fsie {

// ---------------------------------------------------------------- embedding gather
// out[t, :] = table[ids[t], :] widened to the 32-bit residual stream.  An id outside
// [0, vocab) sets *error and yields a row of zeros (the host checks ids first; this is
// the device-side guard the reference kernel lacks, src/cuda/device.cu:41-50).
template <typename T>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                    float* __restrict__ out, int hidden, int vocab, int* error) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) atomicExch(error, 1);
    const T* row = table + (size_t)(ok ? id : 0) * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = ok ? to_float(row[c]) : 0.f;
}

// the same, 8 elements per thread (hidden a multiple of 8)
template <typename T>
__global__ void embed_gather_vec_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                        float* __restrict__ out, int hidden, int vocab, int* error) {
    grid_dependency_wait();
    grid_dependents_go();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) atomicExch(error, 1);
    const T* row = table + (size_t)(ok ? id : 0) * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
        float v[8];
        load8(row + c, v);
        if (!ok) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
        }
        store8(dst + c, v);
    }
}

// ------------------------------------------------------------- add + RMSNorm (fused)
// For output row r (source row s = rows ? rows[r] : r):
//   v = x[s] (+ delta[s]);  if write_x: x[s] = v   (the 32-bit residual sum)
//   y[r] = T( float(v * rsqrt(mean(v^2) + eps)) * gain )
// Formula and order as the reference's rms_norm (src/model/nn.cpp:45-72), with the
// reduction in 32-bit instead of 64-bit.
template <typename T, typename G>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                   const G* __restrict__ gain, T* __restrict__ y,
                                   const int* __restrict__ rows, int hidden, float eps,
                                   int write_x) {
    extern __shared__ float row_cache[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + s * hidden;
    const T* dr = delta ? delta + s * hidden : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = xr[c];
        if (dr) v += to_float(dr[c]);
        row_cache[c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    T* yr = y + (size_t)r * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = row_cache[c];
        if (write_x && dr) xr[c] = v;
        yr[c] = from_float<T>((v * scale) * to_float(gain[c]));
    }
}

// The same with 8 elements per load and the row kept in registers: thread i owns chunks
// i, i + blockDim, ... (NCH of them at most); hidden is a multiple of 8.
template <typename T, typename G, int NCH>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                       const G* __restrict__ gain, T* __restrict__ y,
                                       const int* __restrict__ rows, int hidden, float eps,
                                       int write_x) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    const int chunks = hidden / 8;
    // the gain and the list of rows do not come from the kernel before this one: they are on
    // their way while that kernel still runs (rows of up to 16,384 values: beyond that the
    // registers of the block's up to 1,024 threads do not hold the gain beside the row)
    constexpr bool EARLY_GAIN = NCH <= 2;
    float g[NCH][8];
    if (EARLY_GAIN) {
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < chunks) load8(gain + c * 8, g[k]);
        }
    }
    grid_dependency_wait();
    grid_dependents_go();
    float* xr = x + s * hidden;
    const T* dr = delta ? delta + s * hidden : nullptr;
    float v[NCH][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < chunks) {
            load8(xr + c * 8, v[k]);
            if (dr) {
                float d[8];
                load8(dr + c * 8, d);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[k][i] += d[i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += v[k][i] * v[k][i];
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    T* yr = y + (size_t)r * hidden;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < chunks) {
            if (write_x && dr) store8(xr + c * 8, v[k]);
            float o[8];
            if (!EARLY_GAIN) load8(gain + c * 8, g[k]);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = (v[k][i] * scale) * g[k][i];
            store8(yr + c * 8, o);
        }
    }
}

// ----------------------------------------------- rotary encoding + paged cache write
// One block per token.  q is rotated in place inside the fused projection buffer
// [tokens, ld]; k is rotated and written to its slot of the key pages; v is copied to
// the value pages.  Pairing (i, i + rotary_dim/2) and formula as the reference's
// rope_inplace (src/model/nn.cpp:110-149); cos and sin come from a table the host
// computed in 64-bit.  Dimensions at or beyond rotary_dim pass through unrotated.
// Page layout: [page][kv_head][slot][head_dim]; slot_of[t] = page * page_size + offset,
// or -1 when this token's keys are not to be stored.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int ld, const int* __restrict__ positions,
                                     const float* __restrict__ cos_sin, int table_len,
                                     const int* __restrict__ slot_of,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     long long page_stride, int page_size,
                                     int heads, int kv_heads, int head_dim, int rotary_dim,
                                     int write_cache, int* error) {
    const int t = blockIdx.x;
    int pos = positions[t];
    if (rotary_dim > 0 && (pos < 0 || pos >= table_len)) {
        if (threadIdx.x == 0) atomicExch(error, 2);
        pos = 0;
    }
    const int half = rotary_dim / 2;
    const float* cs = cos_sin + (size_t)pos * rotary_dim;   // [cos(half) | sin(half)]
    T* row = qkv + (size_t)t * ld;
    const int q_width = heads * head_dim, kv_width = kv_heads * head_dim;
    const int hd2 = head_dim / 2;

    // q: rotate in place (each thread owns one pair, or one pass-through pair)
    for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        T* head = row + h * head_dim;
        const float c = cs[i], s = cs[half + i];
        const float x1 = to_float(head[i]), x2 = to_float(head[i + half]);
        head[i] = from_float<T>(x1 * c - x2 * s);
        head[i + half] = from_float<T>(x2 * c + x1 * s);
    }
    (void)hd2;
    if (!write_cache) return;
    const int slot = slot_of[t];
    if (slot < 0) return;
    const long long page = slot / page_size;
    const int offset = slot - (int)page * page_size;
    T* kdst = k_pages + page * page_stride;
    T* vdst = v_pages + page * page_stride;
    const T* krow = row + q_width;
    const T* vrow = row + q_width + kv_width;
    for (int idx = threadIdx.x; idx < kv_width; idx += blockDim.x) {
        const int h = idx / head_dim, d = idx - h * head_dim;
        const size_t dst = ((size_t)h * page_size + offset) * head_dim + d;
        float kv;
        if (d < half) {
            const float c = cs[d], s = cs[half + d];
            kv = to_float(krow[idx]) * c - to_float(krow[idx + half]) * s;
        } else if (d < rotary_dim) {
            const int i = d - half;
            const float c = cs[i], s = cs[half + i];
            kv = to_float(krow[idx]) * c + to_float(krow[idx - half]) * s;
        } else {
            kv = to_float(krow[idx]);
        }
        kdst[dst] = from_float<T>(kv);
        vdst[dst] = vrow[idx];
    }
}

// The same work in chunks of 8 elements, one chunk (or chunk pair) per thread and pass.
// Needs head_dim, rotary_dim / 2 and ld multiples of 8.  Work items of a token, in order:
//   heads * hc         q pairs: chunk i of the first half with chunk i of the second half
//   kv_heads * hc      k pairs, rotated and stored
//   kv_heads * pc      k chunks beyond rotary_dim, stored as they are
//   kv_heads * dc      v chunks, stored                (hc = rotary_dim/16, pc = (head_dim - rotary_dim)/8, dc = head_dim/8)
template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, int ld, const int* __restrict__ positions,
                                         const float* __restrict__ cos_sin, int table_len,
                                         const int* __restrict__ slot_of,
                                         T* __restrict__ k_pages, T* __restrict__ v_pages,
                                         long long page_stride, int page_size,
                                         int heads, int kv_heads, int head_dim, int rotary_dim,
                                         int write_cache, int* error) {
    // The token's position and slot were staged before the step and the table is a constant: they,
    // and the angles of the first rotation item of each thread, are fetched while the kernel
    // before this one (the q,k,v product) still runs.
    const int t = blockIdx.x;
    int pos = positions[t];
    const bool refused = rotary_dim > 0 && (pos < 0 || pos >= table_len);
    if (refused) pos = 0;
    const int half = rotary_dim / 2, hc = half / 8, pc = (head_dim - rotary_dim) / 8, dc = head_dim / 8;
    const float* cs = cos_sin + (size_t)pos * rotary_dim;
    const int q_width = heads * head_dim, kv_width = kv_heads * head_dim;
    const int slot = write_cache ? slot_of[t] : -1;
    const bool store = slot >= 0;
    const int n_q = heads * hc, n_k = kv_heads * hc, n_p = kv_heads * pc, n_v = kv_heads * dc;
    const int total = n_q + (store ? n_k + n_p + n_v : 0);
    float c_first[8], s_first[8];
    if ((int)threadIdx.x < n_q + n_k && (int)threadIdx.x < total) {
        const int w = (int)threadIdx.x < n_q ? threadIdx.x : threadIdx.x - n_q;
        const int i = (w % hc) * 8;
        load8(cs + i, c_first);
        load8(cs + half + i, s_first);
    }
    grid_dependency_wait();
    grid_dependents_go();
    if (refused && threadIdx.x == 0) atomicExch(error, 2);
    T* row = qkv + (size_t)t * ld;
    const long long page = store ? slot / page_size : 0;
    const int offset = store ? slot - (int)page * page_size : 0;
    T* kdst = k_pages + page * page_stride;
    T* vdst = v_pages + page * page_stride;
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        if (idx < n_q + n_k) {
            const bool is_q = idx < n_q;
            const int w = is_q ? idx : idx - n_q;
            const int h = w / hc, i = (w - h * hc) * 8;
            T* head = row + (is_q ? 0 : q_width) + h * head_dim;
            float a[8], b[8], c[8], s[8], lo[8], hi[8];
            load8(head + i, a);
            load8(head + half + i, b);
            if (idx == (int)threadIdx.x) {
#pragma unroll
                for (int e = 0; e < 8; ++e) { c[e] = c_first[e]; s[e] = s_first[e]; }
            } else {
                load8(cs + i, c);
                load8(cs + half + i, s);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                lo[e] = a[e] * c[e] - b[e] * s[e];
                hi[e] = b[e] * c[e] + a[e] * s[e];
            }
            if (is_q) {
                store8(head + i, lo);
                store8(head + half + i, hi);
            } else {
                T* dst = kdst + ((size_t)h * page_size + offset) * head_dim;
                store8(dst + i, lo);
                store8(dst + half + i, hi);
            }
        } else if (idx < n_q + n_k + n_p) {
            const int w = idx - n_q - n_k;
            const int h = w / pc, i = rotary_dim + (w - h * pc) * 8;
            float a[8];
            load8(row + q_width + h * head_dim + i, a);
            store8(kdst + ((size_t)h * page_size + offset) * head_dim + i, a);
        } else {
            const int w = idx - n_q - n_k - n_p;
            const int h = w / dc, i = (w - h * dc) * 8;
            float a[8];
            load8(row + q_width + kv_width + h * head_dim + i, a);
            store8(vdst + ((size_t)h * page_size + offset) * head_dim + i, a);
        }
    }
}

// --------------------------------------------------------------------------- SwiGLU
// act[t, i] = silu(gate[t, i]) * up[t, i] with gate = gu[t, i], up = gu[t, inter + i];
// silu(g) = g / (1 + exp(-g)) in 32-bit as the reference (src/model/nn.cpp:74-88).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter,
                              long long total) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_float(gu[t * 2 * inter + i]);
    const float u = to_float(gu[t * 2 * inter + inter + i]);
    act[idx] = from_float<T>((g / (1.0f + expf(-g))) * u);
}

// 8 elements per thread (inter a multiple of 8)
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter,
                                  long long chunks) {
    grid_dependency_wait();
    grid_dependents_go();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= chunks) return;
    const int per_row = inter / 8;
    const long long t = idx / per_row;
    const int i = (int)(idx - t * per_row) * 8;
    float g[8], u[8], o[8];
    load8(gu + t * 2 * inter + i, g);
    load8(gu + t * 2 * inter + inter + i, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = (g[e] / (1.0f + expf(-g[e]))) * u[e];
    store8(act + t * inter + i, o);
}

// --------------------------------------------------------------------------- token feedback
// ids[dst[i]] = chosen[row[i]]: tokens that the step before sampled enter this step's ids on
// the device, before the host has seen them.
__global__ void place_tokens_kernel(int* __restrict__ ids, const int* __restrict__ dst,
                                    const int* __restrict__ row, const int* __restrict__ chosen, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ids[dst[i]] = chosen[row[i]];
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_embed_gather(const int* ids, const void* table, float* out, int tokens, int hidden,
                      int vocab, int dtype, int* error, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (hidden % 8 == 0) {
        const int threads = hidden / 8 >= 256 ? 256 : (hidden / 8 >= 128 ? 128 : 64);
        if (dtype == DTYPE_F32)
            return launch_dependent(embed_gather_vec_kernel<float>, tokens, threads, 0, stream, ids, (const float*)table, out, hidden, vocab, error);
        return launch_dependent(embed_gather_vec_kernel<bf16>, tokens, threads, 0, stream, ids, (const bf16*)table, out, hidden, vocab, error);
    }
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == DTYPE_F32)
        embed_gather_kernel<float><<<tokens, threads, 0, stream>>>(ids, (const float*)table, out, hidden, vocab, error);
    else
        embed_gather_kernel<bf16><<<tokens, threads, 0, stream>>>(ids, (const bf16*)table, out, hidden, vocab, error);
    return FSIE_LAUNCH_CHECK();
}

int fsie_add_rmsnorm(float* x, const void* delta, const void* gain, int gain_is_f32, void* y,
                     const int* rows, int num_rows, int hidden, float eps, int write_x, int dtype,
                     cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (hidden % 8 == 0 && hidden / 8 <= 4096) {
        // one chunk of 8 per thread up to 1024 chunks, then 2 or 4 chunks per thread
        const int chunks = hidden / 8;
        const int nch = chunks <= 1024 ? 1 : (chunks <= 2048 ? 2 : 4);
        const int threads = ((chunks + nch - 1) / nch + 31) / 32 * 32;
#define FSIE_NORM_VEC(T, G)                                                                      \
        (nch == 1 ? launch_dependent(add_rmsnorm_vec_kernel<T, G, 1>, num_rows, threads, 0, stream, \
                                     x, (const T*)delta, (const G*)gain, (T*)y, rows, hidden, eps, write_x) \
         : nch == 2 ? launch_dependent(add_rmsnorm_vec_kernel<T, G, 2>, num_rows, threads, 0, stream, \
                                       x, (const T*)delta, (const G*)gain, (T*)y, rows, hidden, eps, write_x) \
                    : launch_dependent(add_rmsnorm_vec_kernel<T, G, 4>, num_rows, threads, 0, stream, \
                                       x, (const T*)delta, (const G*)gain, (T*)y, rows, hidden, eps, write_x))
        if (dtype == DTYPE_F32) return FSIE_NORM_VEC(float, float);
        if (gain_is_f32) return FSIE_NORM_VEC(bf16, float);
        return FSIE_NORM_VEC(bf16, bf16);
#undef FSIE_NORM_VEC
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return ERR_UNSUPPORTED;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
#define FSIE_NORM(T, G)                                                                          \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(add_rmsnorm_kernel<T, G>,                                       \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        add_rmsnorm_kernel<T, G><<<num_rows, threads, smem, stream>>>(                           \
            x, (const T*)delta, (const G*)gain, (T*)y, rows, hidden, eps, write_x);              \
    } while (0)
    if (dtype == DTYPE_F32) {
        FSIE_NORM(float, float);
    } else if (gain_is_f32) {
        FSIE_NORM(bf16, float);
    } else {
        FSIE_NORM(bf16, bf16);
    }
#undef FSIE_NORM
    return FSIE_LAUNCH_CHECK();
}

int fsie_rope_kv_write(void* qkv, int ld, const int* positions, const float* cos_sin, int table_len,
                       const int* slot_of, void* k_pages, void* v_pages, long long page_stride,
                       int page_size, int tokens, int heads, int kv_heads, int head_dim,
                       int rotary_dim, int write_cache, int dtype, int* error, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return ERR_BAD_ARGUMENT;
    if (head_dim % 8 == 0 && rotary_dim % 16 == 0 && ld % 8 == 0 && page_stride % 8 == 0) {
        const int items = (heads + kv_heads) * (rotary_dim / 16) + kv_heads * ((head_dim - rotary_dim) / 8) +
                          kv_heads * (head_dim / 8);
        const int vthreads = items >= 512 ? 512 : (items + 31) / 32 * 32;
        if (dtype == DTYPE_F32)
            return launch_dependent(rope_kv_write_vec_kernel<float>, tokens, vthreads, 0, stream,
                (float*)qkv, ld, positions, cos_sin, table_len, slot_of, (float*)k_pages, (float*)v_pages,
                page_stride, page_size, heads, kv_heads, head_dim, rotary_dim, write_cache, error);
        return launch_dependent(rope_kv_write_vec_kernel<bf16>, tokens, vthreads, 0, stream,
            (bf16*)qkv, ld, positions, cos_sin, table_len, slot_of, (bf16*)k_pages, (bf16*)v_pages,
            page_stride, page_size, heads, kv_heads, head_dim, rotary_dim, write_cache, error);
    }
    const int threads = 256;
    if (dtype == DTYPE_F32)
        rope_kv_write_kernel<float><<<tokens, threads, 0, stream>>>(
            (float*)qkv, ld, positions, cos_sin, table_len, slot_of, (float*)k_pages, (float*)v_pages,
            page_stride, page_size, heads, kv_heads, head_dim, rotary_dim, write_cache, error);
    else
        rope_kv_write_kernel<bf16><<<tokens, threads, 0, stream>>>(
            (bf16*)qkv, ld, positions, cos_sin, table_len, slot_of, (bf16*)k_pages, (bf16*)v_pages,
            page_stride, page_size, heads, kv_heads, head_dim, rotary_dim, write_cache, error);
    return FSIE_LAUNCH_CHECK();
}

int fsie_swiglu(const void* gu, void* act, long long tokens, int inter, int dtype,
                cudaStream_t stream) {
    const long long total = tokens * inter;
    if (total <= 0) return 0;
    const int threads = 256;
    if (inter % 8 == 0) {
        const long long chunks = total / 8;
        const unsigned vblocks = (unsigned)((chunks + threads - 1) / threads);
        if (dtype == DTYPE_F32)
            return launch_dependent(swiglu_vec_kernel<float>, vblocks, threads, 0, stream, (const float*)gu, (float*)act, inter, chunks);
        return launch_dependent(swiglu_vec_kernel<bf16>, vblocks, threads, 0, stream, (const bf16*)gu, (bf16*)act, inter, chunks);
    }
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == DTYPE_F32)
        swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)act, inter, total);
    else
        swiglu_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)act, inter, total);
    return FSIE_LAUNCH_CHECK();
}

int fsie_place_tokens(int* ids, const int* dst, const int* row, const int* chosen, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    place_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(ids, dst, row, chosen, n);
    return FSIE_LAUNCH_CHECK();
}

}  // extern "C"
