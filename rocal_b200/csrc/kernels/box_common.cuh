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

}  // namespace rb200
