// Merge of split key ranges for the bfloat16 attention kernels (attention_mma.cu,
// attention_tcgen05.cu).  Needs HD (head size) defined before inclusion.
#pragma once

namespace fsie {

// Merge the key splits of one (token, head); same arithmetic as attention_generic.cu.  The
// weights e^(m_z - M) of splits z and z + 32 are computed once by lane z (nsplit <= 64) and
// broadcast.
constexpr int MAX_KEY_SPLITS = 64;
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                        bf16* __restrict__ out, int out_ld, int tokens, int heads,
                                        int nsplit, const int* __restrict__ token_list) {
    // the list of tokens was staged before the step: it is read while the attention kernel still runs
    const int tok = token_list ? token_list[blockIdx.x] : blockIdx.x, h = blockIdx.y;
    grid_dependency_wait();
    grid_dependents_go();
    const int lane = threadIdx.x & 31;
    const size_t stride = (size_t)tokens * heads;              // (token, head) slots per split
    const size_t slot = (size_t)tok * heads + h;
    float mz = -INFINITY, lz = 0.f, mz_hi = -INFINITY, lz_hi = 0.f;
    if (lane < nsplit) {
        mz = part_ml[(lane * stride + slot) * 2];
        lz = part_ml[(lane * stride + slot) * 2 + 1];
    }
    if (lane + 32 < nsplit) {
        mz_hi = part_ml[((lane + 32) * stride + slot) * 2];
        lz_hi = part_ml[((lane + 32) * stride + slot) * 2 + 1];
    }
    // the first eight splits' values are asked for at once, beside the maxima and sums above: their
    // addresses do not depend on those (one trip to memory instead of two in a row)
    const int d_first = threadIdx.x * 2;
    float2 ahead[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int z = min(j, nsplit - 1);
        ahead[j] = d_first < HD ? *reinterpret_cast<const float2*>(part_o + (z * stride + slot) * HD + d_first)
                                : make_float2(0.f, 0.f);
    }
    const float mmax = warp_max(fmaxf(mz, mz_hi));
    const float wz = mz == -INFINITY ? 0.f : __expf(mz - mmax);
    const float wz_hi = mz_hi == -INFINITY ? 0.f : __expf(mz_hi - mmax);
    const float denom = warp_sum(lz * wz + lz_hi * wz_hi);
    const float inv = denom > 0.f ? 1.0f / denom : 0.f;
    // every lane of a warp takes every turn of this loop (the weights travel by shuffles); lanes
    // beyond the head's end - head sizes that are no multiple of 64 - load and store nothing
    for (int d0 = 0; d0 < HD; d0 += blockDim.x * 2) {
        const int d = d0 + threadIdx.x * 2;
        const bool mine = d < HD;
        float a0 = 0.f, a1 = 0.f;
        for (int z0 = 0; z0 < nsplit; z0 += 8) {
            // eight splits' values are asked for before the first is used: one trip to memory for
            // eight, not eight trips
            float2 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int z = min(z0 + j, nsplit - 1);
                if (d0 == 0 && z0 == 0) v[j] = ahead[j];
                else v[j] = mine ? *reinterpret_cast<const float2*>(part_o + (z * stride + slot) * HD + d)
                                 : make_float2(0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int z = min(z0 + j, MAX_KEY_SPLITS - 1);
                const float lo = __shfl_sync(0xffffffffu, wz, z & 31), hi = __shfl_sync(0xffffffffu, wz_hi, z & 31);
                const float w = z < 32 ? lo : hi;
                if (z0 + j < nsplit && w != 0.f) { a0 += v[j].x * w; a1 += v[j].y * w; }   // a split without keys may hold anything
            }
        }
        if (mine)
            *reinterpret_cast<__nv_bfloat162*>(out + (size_t)tok * out_ld + h * HD + d) =
                __floats2bfloat162_rn(a0 * inv, a1 * inv);
    }
}

}  // namespace fsie
