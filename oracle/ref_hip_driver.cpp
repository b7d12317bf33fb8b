/*
 * ref_hip_driver.cpp — C entry points around the reference's own pixel kernels. TEST INFRASTRUCTURE ONLY.
 *
 * Built by oracle/build.py together with rocAL/rocAL_hip/rocal_hip_kernels.cpp, which is compiled for the
 * host where it lies in the reference tree against the stand-in headers in ref_stubs/hip/ (nothing of the
 * reference is copied). The result, oracle/_ref/libref_hip.so, runs the reference's device code thread by
 * thread on the CPU and pins the pixel arithmetic of the restatement in oracle.c:
 *
 *   ref_hip_resize_bilinear_pkd3 -> HipExecResizeTensor, channels = 3 -> resize_bilinear_pkd_hip_tensor
 *                                   (rocal_hip_kernels.cpp:446-485, helpers :311-444)
 *   ref_hip_resize_generic_pln1  -> HipExecResizeTensor, channels = 1 -> resize_generic_pln1_hip_tensor
 *                                   (rocal_hip_kernels.cpp:487-589)
 *   ref_hip_copy_int8            -> HipExecCopyInt8ToNHWC / HipExecCopyInt8ToNCHW and the four
 *                                   Hip_CopyInt8To* converters (rocal_hip_kernels.cpp:40-309)
 *
 * The bilinear kernel stores 8 pixels per thread whatever the sample's width and loads 4 bytes per 3-byte
 * pixel, so this driver runs it on private buffers with slack (rows padded to a multiple of 8 pixels plus
 * 8) and copies the valid region out.
 */
#include <cstdint>
#include <cstring>
#include <vector>

#include "hip/hip_runtime.h"
#include "rocal_hip_kernels.h"

#define REF_API extern "C" __attribute__((visibility("default")))

/* src: n images, image i = src_h[i] rows of src_stride[i] bytes at src + src_offset[i] (uint8 RGB interleaved).
 * dst: [n][max_dst_h][max_dst_w][3]; only dst_h[i] x dst_w[i] of sample i is written, the rest is left as found. */
REF_API int ref_hip_resize_bilinear_pkd3(const uint8_t* src, size_t src_bytes, int n, const uint32_t* src_w,
                                         const uint32_t* src_h, const uint32_t* src_stride, const uint64_t* src_offset,
                                         const uint32_t* dst_w, const uint32_t* dst_h, uint32_t max_dst_w,
                                         uint32_t max_dst_h, uint8_t* dst) {
    std::vector<uint8_t> in(src_bytes + 64, 0);
    memcpy(in.data(), src, src_bytes);
    const size_t pad_w = ((size_t)max_dst_w + 7) / 8 * 8 + 8;
    std::vector<uint8_t> out((size_t)n * max_dst_h * pad_w * 3 + 64, 0);
    std::vector<size_t> sw(n), sh(n), dw(n), dh(n), ss(n), so(n);
    size_t max_sw = 0, max_sh = 0;
    for (int i = 0; i < n; i++) {
        sw[i] = src_w[i]; sh[i] = src_h[i]; dw[i] = dst_w[i]; dh[i] = dst_h[i]; ss[i] = src_stride[i]; so[i] = src_offset[i];
        if (sw[i] > max_sw) max_sw = sw[i];
        if (sh[i] > max_sh) max_sh = sh[i];
    }
    HipExecResizeTensor(nullptr, in.data(), out.data(), (unsigned)n, sw.data(), sh.data(), dw.data(), dh.data(), ss.data(),
                        so.data(), 3, max_sw, max_sh, pad_w, max_dst_h);
    for (int i = 0; i < n; i++)
        for (uint32_t y = 0; y < dst_h[i] && y < max_dst_h; y++)
            memcpy(dst + (((size_t)i * max_dst_h + y) * max_dst_w) * 3, out.data() + (((size_t)i * max_dst_h + y) * pad_w) * 3,
                   (size_t)(dst_w[i] < max_dst_w ? dst_w[i] : max_dst_w) * 3);
    return 0;
}

/* Single-channel planes: image i = src_h[i] rows of src_stride[i] bytes at src + src_offset[i]; dst [n][max_dst_h][max_dst_w]. */
REF_API int ref_hip_resize_generic_pln1(const uint8_t* src, size_t src_bytes, int n, const uint32_t* src_w,
                                        const uint32_t* src_h, const uint32_t* src_stride, const uint64_t* src_offset,
                                        const uint32_t* dst_w, const uint32_t* dst_h, uint32_t max_dst_w,
                                        uint32_t max_dst_h, uint8_t* dst) {
    std::vector<uint8_t> in(src_bytes + 64, 0);
    memcpy(in.data(), src, src_bytes);
    std::vector<size_t> sw(n), sh(n), dw(n), dh(n), ss(n), so(n);
    size_t max_sw = 0, max_sh = 0;
    for (int i = 0; i < n; i++) {
        sw[i] = src_w[i]; sh[i] = src_h[i]; dw[i] = dst_w[i]; dh[i] = dst_h[i]; ss[i] = src_stride[i]; so[i] = src_offset[i];
        if (sw[i] > max_sw) max_sw = sw[i];
        if (sh[i] > max_sh) max_sh = sh[i];
    }
    HipExecResizeTensor(nullptr, in.data(), dst, (unsigned)n, sw.data(), sh.data(), dw.data(), dh.data(), ss.data(), so.data(), 1,
                        max_sw, max_sh, max_dst_w, max_dst_h);
    return 0;
}

/* src: [n][h][w][3] uint8; out: nchw != 0 ? [n][3][h][w] : [n][h][w][3], float32 or (fp16 != 0) half. */
REF_API int ref_hip_copy_int8(const uint8_t* src, int n, int h, int w, int nchw, int fp16, const float* mul, const float* add,
                              int reverse_channels, void* out) {
    if (nchw)
        return HipExecCopyInt8ToNCHW(nullptr, src, out, 0, n, 3, h, w, mul[0], mul[1], mul[2], add[0], add[1], add[2],
                                     reverse_channels, fp16, 0, 0);
    return HipExecCopyInt8ToNHWC(nullptr, src, out, 0, n, 3, h, w, mul[0], mul[1], mul[2], add[0], add[1], add[2],
                                 reverse_channels, fp16, 0, 0);
}
