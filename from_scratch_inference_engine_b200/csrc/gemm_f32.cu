// True 32-bit matrix products for the float32 path: y[M,N] = x[M,K] * w[N,K]^T (+ bias[N]).
// Plain FFMA on CUDA cores, no tensor-core mode of any precision (the reference instead asks
// its library for strict fp32, src/cuda/device.cu:322-357).  Three kernels:
//
//  * gemm_f32_rows_kernel - steps of few tokens (M <= 48, in tiles of up to 16 rows).  The
//    product is bound by reading w once from HBM, so a warp owns R rows of w and streams them
//    with 16-byte loads, its 32 lanes side by side along k; the step's rows of x wait in shared
//    memory and every x value read from there is used for R rows of w.  A lane's partial sums
//    run over k in ascending order and the 32 lanes are then added in a fixed tree, so an
//    output does not depend on how many other rows share the launch.
//  * gemm_f32_tiles_kernel - prompts: tiles of 128 x 128 outputs, k in steps of 16 through
//    shared memory, 8 x 8 outputs per thread in registers.  Each output is one thread's sum over
//    k in ascending order.
//  * gemm_f32_plain_kernel - any sizes and alignments (k no multiple of 4, unaligned rows).
//
// An output of the rows kernel and the same output of the tiles kernel differ in the order of
// their sums, that is by rounding; within one kernel a row's result does not depend on the batch.
#include "common.cuh"

namespace fsie {

// ------------------------------------------------------------------------- few rows
constexpr int ROWS_WARPS = 8;        // warps per block

// 16 bytes from global to shared memory without passing through registers; src_bytes = 0 writes zeros.
__device__ __forceinline__ void copy16_async(void* dst, const void* src, int src_bytes) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void copies_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// MT rows of x per block, R rows of w per warp.  A warp walks k in passes of 128 elements (16
// bytes per lane and row of w) and keeps the rows of w of the next DEPTH - 1 passes on their
// way into registers while it multiplies the current one, so that its requests to HBM never
// pause.  The step's rows of x come through shared memory in chunks of XC elements, the next
// chunk copied (without registers) while the current one is used: one barrier per chunk.
constexpr int ROWS_DEPTH = 4;
template <int MT> struct RowsChunk { static constexpr int XC = MT >= 16 ? 512 : 1024; };

template <int MT, int R, bool EXACT>      // EXACT: K is a multiple of 128, no pass has a ragged end
__global__ void __launch_bounds__(ROWS_WARPS * 32, MT * R <= 32 ? 2 : 1)      // two blocks per SM unless the sums alone need 64 registers
gemm_f32_rows_kernel(const float* __restrict__ x, const float* __restrict__ w,
                     const float* __restrict__ bias, float* __restrict__ y,
                     int M, int N, int K, int ldx, int ldy) {
    constexpr int XC = RowsChunk<MT>::XC, PER_CHUNK = XC / 128, D = ROWS_DEPTH;
    extern __shared__ __align__(16) float xs_raw[];
    float (*xs)[MT][XC] = reinterpret_cast<float (*)[MT][XC]>(xs_raw);       // [2][MT][XC]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the tiles of rows of x are the fast grid dimension: blocks that read the same rows of w
    // run side by side and share them through L2
    const int m0 = blockIdx.x * MT;
    const int n0 = (blockIdx.y * ROWS_WARPS + warp) * R;
    // rows beyond N are computed from the last row and not stored: no warp leaves the loop early,
    // no load or sum below is predicated on it
    const float* wrow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) wrow[r] = w + (size_t)min(n0 + r, N - 1) * K + lane * 4;
    float acc[R][MT];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

    auto stage_x = [&](int chunk) {         // the step's rows of x for one chunk (zeros beyond M and K)
        const int k0 = chunk * XC;
        for (int e = tid; e < MT * (XC / 4); e += ROWS_WARPS * 32) {
            const int m = e / (XC / 4), c = (e - m * (XC / 4)) * 4;
            const bool valid = m0 + m < M && k0 + c < K;
            copy16_async(&xs[chunk & 1][m][c], valid ? x + (size_t)(m0 + m) * ldx + k0 + c : x, valid ? 16 : 0);
        }
    };
    const int passes = (K + 127) / 128;
    auto load_w = [&](int pass, float4 (&dst)[R]) {
        pass = min(pass, passes - 1);       // beyond the end: the last pass again (never multiplied)
        const bool in_range = EXACT || pass * 128 + lane * 4 < K;
#pragma unroll
        for (int r = 0; r < R; ++r)
            dst[r] = in_range ? __ldg(reinterpret_cast<const float4*>(wrow[r] + pass * 128))
                              : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    float4 ring[D][R];
    stage_x(0);
#pragma unroll
    for (int d = 0; d < D - 1; ++d) load_w(d, ring[d]);
    for (int base = 0; base < passes; base += D) {
#pragma unroll
        for (int u = 0; u < D; ++u) {
            const int pass = base + u;
            load_w(pass + D - 1, ring[(u + D - 1) % D]);
            if (pass < passes) {
                const int chunk = pass / PER_CHUNK, within = pass - chunk * PER_CHUNK;
                if (within == 0) {
                    copies_wait_all();
                    __syncthreads();      // this chunk's x has landed, the other half is no longer read
                    if ((chunk + 1) * XC < K) stage_x(chunk + 1);
                }
                const float* xrow = &xs[chunk & 1][0][within * 128 + lane * 4];
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const float4 xv = *reinterpret_cast<const float4*>(xrow + m * XC);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        float a = acc[r][m];
                        a = fmaf(xv.x, ring[u][r].x, a);
                        a = fmaf(xv.y, ring[u][r].y, a);
                        a = fmaf(xv.z, ring[u][r].z, a);
                        a = fmaf(xv.w, ring[u][r].w, a);
                        acc[r][m] = a;
                    }
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float total = warp_sum(acc[r][m]);
            if (lane == 0 && n0 + r < N && m0 + m < M)
                y[(size_t)(m0 + m) * ldy + n0 + r] = total + (bias ? bias[n0 + r] : 0.f);
        }
}

template <int MT, int R>
static int launch_rows_as(const float* x, const float* w, const float* bias, float* y, int M, int N,
                          int K, int ldx, int ldy, int m_tiles, cudaStream_t stream) {
    const size_t smem = sizeof(float) * 2 * MT * RowsChunk<MT>::XC;
    static bool raised = false;          // per instantiation: the limit of dynamic shared memory
    if (!raised && smem > 48 * 1024) {
        if (cudaFuncSetAttribute(gemm_f32_rows_kernel<MT, R, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_f32_rows_kernel<MT, R, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        raised = true;
    }
    const dim3 grid(m_tiles, (N + ROWS_WARPS * R - 1) / (ROWS_WARPS * R));
    if (K % 128 == 0)
        gemm_f32_rows_kernel<MT, R, true><<<grid, ROWS_WARPS * 32, smem, stream>>>(x, w, bias, y, M, N, K, ldx, ldy);
    else
        gemm_f32_rows_kernel<MT, R, false><<<grid, ROWS_WARPS * 32, smem, stream>>>(x, w, bias, y, M, N, K, ldx, ldy);
    return FSIE_LAUNCH_CHECK();
}

template <int MT>
static int launch_rows(const float* x, const float* w, const float* bias, float* y, int M, int N,
                       int K, int ldx, int ldy, int sms, int rows_per_warp, cudaStream_t stream) {
    const int m_tiles = (M + MT - 1) / MT;
    // four rows of w per warp (two from 16 rows of x on, where the sums of four would take 64
    // registers), two where four would leave SMs without two blocks; one row per warp measured
    // slowest at every size (each x value read from shared memory then serves one product only)
    auto blocks = [&](int r) { return (N + ROWS_WARPS * r - 1) / (ROWS_WARPS * r); };
    int r = MT >= 16 ? 2 : 4;
    if (r == 4 && blocks(4) * m_tiles < 2 * sms) r = 2;
    if (rows_per_warp == 1 || rows_per_warp == 2 || rows_per_warp == 4) r = rows_per_warp;
    if (r == 4) return launch_rows_as<MT, 4>(x, w, bias, y, M, N, K, ldx, ldy, m_tiles, stream);
    if (r == 2) return launch_rows_as<MT, 2>(x, w, bias, y, M, N, K, ldx, ldy, m_tiles, stream);
    return launch_rows_as<MT, 1>(x, w, bias, y, M, N, K, ldx, ldy, m_tiles, stream);
}

// ---------------------------------------------------------------------------- tiles
constexpr int TM = 128, TN = 128, TK = 16;      // block tile; 256 threads, 8 x 8 outputs each

__global__ void __launch_bounds__(256, 2)
gemm_f32_tiles_kernel(const float* __restrict__ x, const float* __restrict__ w,
                      const float* __restrict__ bias, float* __restrict__ y,
                      int M, int N, int K, int ldx, int ldy) {
    // k-major in shared memory, so that a thread's 8 rows (columns) are two 16-byte reads
    __shared__ __align__(16) float xs[2][TK][TM + 4];      // + 4: the four k of a thread's load fall into other banks
    __shared__ __align__(16) float ws[2][TK][TN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;           // tx -> columns (N), ty -> rows (M)
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    // loads: 128 rows x 16 k per operand = 512 float4; thread t takes rows t / 4 and t / 4 + 64,
    // k offset (t % 4) * 4
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    float4 xr[2], wr[2];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int m = m0 + lrow + h * 64, n = n0 + lrow + h * 64, k = k0 + lk;
            xr[h] = (m < M && k < K) ? *reinterpret_cast<const float4*>(x + (size_t)m * ldx + k)
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
            wr[h] = (n < N && k < K) ? __ldg(reinterpret_cast<const float4*>(w + (size_t)n * K + k))
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = lrow + h * 64;
            xs[buf][lk + 0][r] = xr[h].x; xs[buf][lk + 1][r] = xr[h].y;
            xs[buf][lk + 2][r] = xr[h].z; xs[buf][lk + 3][r] = xr[h].w;
            ws[buf][lk + 0][r] = wr[h].x; ws[buf][lk + 1][r] = wr[h].y;
            ws[buf][lk + 2][r] = wr[h].z; ws[buf][lk + 3][r] = wr[h].w;
        }
    };
    fetch(0);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int k0 = 0; k0 < K; k0 += TK) {
        const bool more = k0 + TK < K;
        if (more) fetch(k0 + TK);                 // the next step's operands travel while this one computes
#pragma unroll
        for (int c = 0; c < TK; ++c) {
            // rows ty*4 .. +3 and 64 + ty*4 .. +3, columns tx*4 .. +3 and 64 + tx*4 .. +3:
            // consecutive threads read consecutive 16 bytes, no bank conflicts
            const float4 a0 = *reinterpret_cast<const float4*>(&xs[buf][c][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&xs[buf][c][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&ws[buf][c][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&ws[buf][c][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (more) {
            stash(buf ^ 1);
            __syncthreads();
            buf ^= 1;
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
        if (m >= M) continue;
#pragma unroll
        for (int jh = 0; jh < 2; ++jh) {
            const int n = n0 + jh * 64 + tx * 4;
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = acc[i][jh * 4 + j] + ((bias && n + j < N) ? bias[n + j] : 0.f);
            float* out = y + (size_t)m * ldy + n;
            if (n + 3 < N && (((size_t)out) & 15) == 0) {
                *reinterpret_cast<float4*>(out) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (n + j < N) out[j] = v[j];
            }
        }
    }
}

// ---------------------------------------------------------------------------- plain
constexpr int GM = 64, GN = 64, GK = 16;   // block tile; 256 threads, 4x4 outputs each

__global__ void __launch_bounds__(256)
gemm_f32_plain_kernel(const float* __restrict__ x, const float* __restrict__ w,
                      const float* __restrict__ bias, float* __restrict__ y,
                      int M, int N, int K, int ldx, int ldy) {
    __shared__ float xs[GK][GM + 4];
    __shared__ float ws[GK][GN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;           // tx -> columns (N), ty -> rows (M)
    const int m0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GK) {
        // 64x16 elements per operand, 256 threads -> 4 each; consecutive threads walk k
        for (int e = tid; e < GM * GK; e += 256) {
            const int r = e / GK, c = e - r * GK;
            const int m = m0 + r, n = n0 + r, k = k0 + c;
            xs[c][r] = (m < M && k < K) ? x[(size_t)m * ldx + k] : 0.f;
            ws[c][r] = (n < N && k < K) ? w[(size_t)n * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < GK; ++c) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[c][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[c][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) y[(size_t)m * ldy + n] = acc[i][j] + (bias ? bias[n] : 0.f);
        }
    }
}

}  // namespace fsie

// Rows of a step that still take the few-rows kernel (in tiles of 16).  Measured on the
// 37,888 x 3,584 matrix: 32 rows 0.46 ms against 0.79 ms for the tiles kernel, 64 rows 0.88
// against 0.79 - the tiles kernel's time does not depend on the rows below 128.
extern "C" int fsie_gemm_f32_rows_limit() { return 48; }

// kind: 0 = choose by size and alignment, 1 = few-rows kernel, 2 = tiles kernel, 3 = plain kernel
// (the tests ask for each by name; a kind that cannot take the operands is refused).
// rows_per_warp: 0 = chosen by size; 1, 2 or 4 fix it for the few-rows kernel (tests, measurements).
extern "C" int fsie_gemm_f32(const float* x, const float* w, const float* bias, float* y, int M,
                             int N, int K, int ldx, int ldy, int kind, int rows_per_warp,
                             cudaStream_t stream) {
    using namespace fsie;
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || kind < 0 || kind > 3) return ERR_BAD_ARGUMENT;
    // 16-byte loads need k in steps of 4 and rows that start on 16 bytes
    const bool aligned = (K % 4 == 0) && (ldx % 4 == 0) && ((((size_t)x) | ((size_t)w)) & 15) == 0;
    if ((kind == 1 || kind == 2) && !aligned) return ERR_UNSUPPORTED;
    if (kind == 1 && M > fsie_gemm_f32_rows_limit()) return ERR_UNSUPPORTED;
    if (kind == 0) kind = !aligned ? 3 : (M <= fsie_gemm_f32_rows_limit() ? 1 : 2);
    if (kind == 3) {
        dim3 grid((N + GN - 1) / GN, (M + GM - 1) / GM);
        gemm_f32_plain_kernel<<<grid, 256, 0, stream>>>(x, w, bias, y, M, N, K, ldx, ldy);
        return FSIE_LAUNCH_CHECK();
    }
    if (kind == 2) {
        dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
        gemm_f32_tiles_kernel<<<grid, 256, 0, stream>>>(x, w, bias, y, M, N, K, ldx, ldy);
        return FSIE_LAUNCH_CHECK();
    }
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (M == 1) return launch_rows<1>(x, w, bias, y, M, N, K, ldx, ldy, sms, rows_per_warp, stream);
    if (M == 2) return launch_rows<2>(x, w, bias, y, M, N, K, ldx, ldy, sms, rows_per_warp, stream);
    if (M <= 4) return launch_rows<4>(x, w, bias, y, M, N, K, ldx, ldy, sms, rows_per_warp, stream);
    if (M <= 8) return launch_rows<8>(x, w, bias, y, M, N, K, ldx, ldy, sms, rows_per_warp, stream);
    return launch_rows<16>(x, w, bias, y, M, N, K, ldx, ldy, sms, rows_per_warp, stream);
}
