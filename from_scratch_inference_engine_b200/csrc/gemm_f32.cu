// True 32-bit matrix product for the float32 path: y[M,N] = x[M,K] * w[N,K]^T (+ bias[N]).
// Plain FFMA on CUDA cores, no tensor-core mode of any precision.  Each output element
// is one thread's sum over k in ascending order, so a row of y does not depend on how
// many other rows share the launch (the reference instead asks its library for strict
// fp32, src/cuda/device.cu:322-357).
#include "common.cuh"

namespace fsie {

constexpr int GM = 64, GN = 64, GK = 16;   // block tile; 256 threads, 4x4 outputs each

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
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

extern "C" int fsie_gemm_f32(const float* x, const float* w, const float* bias, float* y, int M,
                             int N, int K, int ldx, int ldy, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return fsie::ERR_BAD_ARGUMENT;
    dim3 grid((N + fsie::GN - 1) / fsie::GN, (M + fsie::GM - 1) / fsie::GM);
    fsie::gemm_f32_kernel<<<grid, 256, 0, stream>>>(x, w, bias, y, M, N, K, ldx, ldy);
    return FSIE_LAUNCH_CHECK();
}
