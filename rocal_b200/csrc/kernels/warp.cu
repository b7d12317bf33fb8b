// Affine gather (WarpAffine / Rotate): uint8 HWC -> uint8 HWC, bilinear, constant-zero border.
//
// grid = (tiles of the output extent, samples); a CTA owns a 32 x 8 output tile, one thread per
// output pixel, so that the source footprint of a warp stays compact under rotation.
//
// Coordinates: dx = x - (dst_w/2), dy = y - (dst_h/2) (integer halves);
//   sx = fma(m00, dx, fma(m01, dy, t0 + src_w/2)),  sy = fma(m10, dx, fma(m11, dy, t1 + src_h/2)).
// A position whose floor lies outside [0, src-1] gives 0; otherwise both taps are clamped to
// [0, src-2] and blended with the fmaf nest of the bilinear helper in
// rocAL/rocAL_hip/rocal_hip_kernels.cpp:332-343,388-409.
#include "common.cuh"

namespace rb200 {

struct WarpLaunch {
    uint8_t* out;
    int out_w, out_h;
    int tiles_x;
    int fill_padding;
};

__global__ void __launch_bounds__(256) warp_affine_kernel(const uint8_t* __restrict__ arena,
                                                          const rb200_warp_sample* __restrict__ samples,
                                                          const WarpLaunch L) {
    const int n = blockIdx.y;
    const int tx = blockIdx.x % L.tiles_x;
    const int ty = blockIdx.x / L.tiles_x;
    const int x = tx * 32 + (threadIdx.x & 31);
    const int y = ty * 8 + (threadIdx.x >> 5);
    if (x >= L.out_w || y >= L.out_h) return;

    const rb200_warp_sample s = samples[n];
    const uint8_t* img = arena + s.src_offset;
    uint8_t* o = L.out + (((size_t)n * L.out_h + y) * L.out_w + x) * 3;
    const int w = min(s.dst_w, L.out_w), h = min(s.dst_h, L.out_h);
    if (x >= w || y >= h) {
        if (L.fill_padding) { o[0] = 0; o[1] = 0; o[2] = 0; }
        return;
    }
    const float dx = sub_rn((float)x, (float)(s.dst_w / 2));
    const float dy = sub_rn((float)y, (float)(s.dst_h / 2));
    const float t0 = add_rn(s.m[4], mul_rn((float)s.src_w, 0.5f));
    const float t1 = add_rn(s.m[5], mul_rn((float)s.src_h, 0.5f));
    const float sx = fmaf(s.m[0], dx, fmaf(s.m[1], dy, t0));
    const float sy = fmaf(s.m[2], dx, fmaf(s.m[3], dy, t1));
    const float fx = floorf(sx), fy = floorf(sy);
    float v0 = 0.f, v1 = 0.f, v2 = 0.f;
    // Written so that NaN coordinates fall through to the interpolation exactly as in the checker.
    if (!(fx < 0.f || fy < 0.f || fx > (float)(s.src_w - 1) || fy > (float)(s.src_h - 1))) {
        const float wx = sub_rn(sx, fx), wy = sub_rn(sy, fy);
        const float owx = sub_rn(1.0f, wx), owy = sub_rn(1.0f, wy);
        const int xh = max(s.src_w - 2, 0), yh = max(s.src_h - 2, 0);
        const int x0 = (int)fminf(fmaxf(fx, 0.f), (float)xh);
        const int y0 = (int)fminf(fmaxf(fy, 0.f), (float)yh);
        const int x1 = (int)fminf(fmaxf(add_rn(fx, 1.0f), 0.f), (float)xh);
        const int y1 = (int)fminf(fmaxf(add_rn(fy, 1.0f), 0.f), (float)yh);
        const uint8_t* r0 = img + (size_t)y0 * s.src_stride;
        const uint8_t* r1 = img + (size_t)y1 * s.src_stride;
        const float w00 = mul_rn(owy, owx), w01 = mul_rn(owy, wx), w10 = mul_rn(wy, owx);
        float v[3];
#pragma unroll
        for (int c = 0; c < 3; c++) {
            float tl = (float)__ldg(r0 + x0 * 3 + c), tr = (float)__ldg(r0 + x1 * 3 + c);
            float bl = (float)__ldg(r1 + x0 * 3 + c), br = (float)__ldg(r1 + x1 * 3 + c);
            float acc = mul_rn(mul_rn(br, wy), wx);
            acc = fmaf(bl, w10, acc);
            acc = fmaf(tr, w01, acc);
            acc = fmaf(tl, w00, acc);
            v[c] = sat_round_u8f(acc);
        }
        v0 = v[0]; v1 = v[1]; v2 = v[2];
    }
    o[0] = (uint8_t)v0;
    o[1] = (uint8_t)v1;
    o[2] = (uint8_t)v2;
}

}  // namespace rb200

using namespace rb200;

extern "C" int rb200k_warp_affine(const uint8_t* arena, const rb200_warp_sample* samples, int n,
                                  const rb200_warp_params* p, void* stream_v) {
    if (n == 0) return RB200_OK;
    if (!arena || !samples || !p || !p->out || n < 0 || p->out_w <= 0 || p->out_h <= 0) {
        set_error("rb200k_warp_affine: null pointer or non-positive size");
        return RB200_E_INVALID;
    }
    if (n > 65535) {
        set_error("rb200k_warp_affine: batch %d exceeds 65535", n);
        return RB200_E_LIMIT;
    }
    WarpLaunch L;
    L.out = (uint8_t*)p->out;
    L.out_w = p->out_w;
    L.out_h = p->out_h;
    L.fill_padding = p->fill_padding;
    L.tiles_x = (p->out_w + 31) / 32;
    int tiles_y = (p->out_h + 7) / 8;
    dim3 grid((unsigned)(L.tiles_x * tiles_y), (unsigned)n);
    warp_affine_kernel<<<grid, 256, 0, (cudaStream_t)stream_v>>>(arena, samples, L);
    RB200_CHECK_LAUNCH("warp_affine_kernel");
    return RB200_OK;
}
