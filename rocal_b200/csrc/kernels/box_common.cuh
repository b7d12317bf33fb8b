// Shared by the SSD box encoder and the box IoU matcher.
#pragma once
#include "common.cuh"

namespace rb200 {

// IoU of two ltrb boxes as the CPU code computes it (rocAL/source/meta_data/bounding_box_graph.cpp:61-69):
// inter / (area_b + area_a - inter), float32, one rounding per operation.
__device__ __forceinline__ float iou_ltrb(const float4 b, float area_b, const float4 a, float area_a) {
    float xa = fmaxf(b.x, a.x), ya = fmaxf(b.y, a.y);
    float xb = fminf(b.z, a.z), yb = fminf(b.w, a.w);
    float inter = mul_rn(fmaxf(0.f, sub_rn(xb, xa)), fmaxf(0.f, sub_rn(yb, ya)));
    float uni = sub_rn(add_rn(area_b, area_a), inter);
    // Most box/anchor pairs do not overlap. 0 / u is a zero for every non-zero, non-NaN u, and the IEEE
    // division of a zero numerator takes the slow path of the division sequence, so it is answered here;
    // the sign of that zero never matters to the comparisons that consume the value.
    if (inter == 0.f && (uni > 0.f || uni < 0.f)) return 0.f;
    return div_rn(inter, uni);
}

// Order-preserving map of a non-NaN float onto unsigned integers, and back.
__device__ __forceinline__ uint32_t float_key(float v) {
    const uint32_t bits = __float_as_uint(v);
    return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

constexpr int kOrderMax = 512;  // batches up to this size are processed longest sample first

// Which sample this cluster takes. A cluster's life is proportional to its sample's box count (1..50 in SSD training),
// and clusters are handed out in grid order, so taking the samples in their given order leaves the device to a few
// long samples at the end. Up to kOrderMax samples are therefore taken longest first: cluster y finds the sample whose
// box count ranks y-th (ties by index). Every CTA works the small ranking out for itself from the offsets, so no
// scratch memory or extra launch is needed; `cnt` is shared memory of at least kOrderMax ints that is free on entry
// and on return. Kept out of line so that its registers do not add to the main loop's.
static __device__ __noinline__ int pick_sample(const int* __restrict__ box_offsets, int* cnt) {
    const int ns = (int)gridDim.y;
    if (ns <= 1 || ns > kOrderMax) return (int)blockIdx.y;
    __shared__ int s_sample;
    const int tid = threadIdx.x, nthreads = blockDim.x;
    for (int i = tid; i < ns; i += nthreads) cnt[i] = box_offsets[i + 1] - box_offsets[i];
    __syncthreads();
    for (int i = tid; i < ns; i += nthreads) {
        const int c = cnt[i];
        int r = 0;
        for (int j = 0; j < ns; j++) {
            const int cj = cnt[j];
            r += (cj > c || (cj == c && j < i)) ? 1 : 0;
        }
        if (r == (int)blockIdx.y) s_sample = i;
    }
    __syncthreads();
    const int n = s_sample;
    __syncthreads();                        // cnt is free again
    return n;
}

}  // namespace rb200
