// Bilinear resample family: [crop ->] resize [-> crop] [-> mirror] [-> normalize] in one pass.
//
// One launch covers the whole ragged batch: grid = (tiles of the output extent, samples).
// A CTA owns an output tile of TW columns (one thread per column) by TH rows. It first stages
// the source rows its taps touch into shared memory with 16-byte cp.async copies (global
// addresses rounded down to 16 bytes, so every copy is aligned whatever the row pitch of the
// packed uint8 HWC source), then interpolates from shared memory and writes NCHW/NHWC
// fp32/fp16/uint8 directly. Column-dependent values (tap offsets, x weights) are computed once
// per thread and reused for all rows of the tile.
//
// The interpolation follows the reference's HIP bilinear kernel
// (rocAL/rocAL_hip/rocal_hip_kernels.cpp:311-343, 388-409, 425-430): source location
// dst*ratio + (ratio-1)/2 + roi.x, floor, taps clamped to [roi.x, roi.x2-1], the fmaf nest
// TL*(1-wy)(1-wx) + (TR*(1-wy)wx + (BL*wy(1-wx) + BR*wy*wx)), round-to-nearest-even uint8.
#include "common.cuh"

namespace rb200 {

struct ResampleLaunch {
    void* out;
    int out_w, out_h;
    int ext_w, ext_h;   // extent covered by the grid
    int tiles_x;
    int th;             // rows per tile
    int pitch;          // bytes per staged row (multiple of 16)
    int normalize, fill_padding;
    float mul[3], add[3];
};

struct RowInfo {
    float wy, owy;
    int off0, off1;     // staged: byte offset of the row's first staged pixel in shared memory
                        // unstaged: source row index of the two taps
};

__device__ __forceinline__ float src_location(int d, float ratio, float offset, int roi_start) {
    return add_rn(add_rn(mul_rn((float)d, ratio), offset), (float)roi_start);
}

__device__ __forceinline__ void clamp_taps(float f, int lo, int hi, int& t0, int& t1) {
    t0 = (int)fminf(fmaxf(f, (float)lo), (float)hi);
    t1 = (int)fminf(fmaxf(add_rn(f, 1.0f), (float)lo), (float)hi);
}

template <typename OutT, int LAYOUT>
__device__ __forceinline__ void store3(OutT* out, int out_w, int out_h, int n, int y, int x, float v0, float v1, float v2) {
    if (LAYOUT == RB200_NCHW) {
        size_t plane = (size_t)out_w * out_h;
        size_t base = ((size_t)n * 3) * plane + (size_t)y * out_w + x;
        out[base] = OutConv<OutT>::cvt(v0);
        out[base + plane] = OutConv<OutT>::cvt(v1);
        out[base + 2 * plane] = OutConv<OutT>::cvt(v2);
    } else {
        size_t base = (((size_t)n * out_h + y) * out_w + x) * 3;
        out[base] = OutConv<OutT>::cvt(v0);
        out[base + 1] = OutConv<OutT>::cvt(v1);
        out[base + 2] = OutConv<OutT>::cvt(v2);
    }
}

template <typename OutT, int LAYOUT, bool STAGED>
__global__ void __launch_bounds__(256) resample_kernel(const uint8_t* __restrict__ arena,
                                                       const rb200_resample_sample* __restrict__ samples,
                                                       const ResampleLaunch L) {
    extern __shared__ __align__(16) uint8_t smem[];
    // Layout: RowInfo[th] | int srow[2*th+2] | (16-byte aligned) staged rows
    RowInfo* rowinfo = reinterpret_cast<RowInfo*>(smem);
    int* srow = reinterpret_cast<int*>(smem + sizeof(RowInfo) * L.th);
    uint8_t* stage = smem + ((sizeof(RowInfo) * L.th + sizeof(int) * (2 * L.th + 2) + 15) & ~(size_t)15);

    const int n = blockIdx.y;
    const int tx = blockIdx.x % L.tiles_x;
    const int ty = blockIdx.x / L.tiles_x;
    const int tid = threadIdx.x;
    const int TW = blockDim.x;

    const rb200_resample_sample s = samples[n];
    const uint8_t* img = arena + s.src_offset;
    OutT* out = reinterpret_cast<OutT*>(L.out);

    const int cw = min(s.crop_w, L.out_w);
    const int ch = min(s.crop_h, L.out_h);
    const int tile_x0 = tx * TW;
    const int tile_y0 = ty * L.th;
    const int xi = tile_x0 + tid;

    const int rows_valid = min(L.th, ch - tile_y0);     // rows of this tile inside the crop
    const int cols_valid = min(TW, cw - tile_x0);       // columns of this tile inside the crop

    if (rows_valid > 0 && cols_valid > 0) {
        const float ratio_w = div_rn((float)s.roi_w, (float)s.dst_w);
        const float ratio_h = div_rn((float)s.roi_h, (float)s.dst_h);
        const float off_w = mul_rn(sub_rn(ratio_w, 1.0f), 0.5f);
        const float off_h = mul_rn(sub_rn(ratio_h, 1.0f), 0.5f);
        const int x_lo = s.roi_x, y_lo = s.roi_y;
        const int x_hi = max(s.roi_x + s.roi_w - 2, s.roi_x);
        const int y_hi = max(s.roi_y + s.roi_h - 2, s.roi_y);

        // Source column range of the tile (identical in every thread).
        int x_first, x_last;
        {
            int ca = tile_x0, cb = tile_x0 + cols_valid - 1;
            int ra = s.crop_x + (s.mirror ? (s.crop_w - 1 - ca) : ca);
            int rb = s.crop_x + (s.mirror ? (s.crop_w - 1 - cb) : cb);
            int r_lo = min(ra, rb), r_hi = max(ra, rb);
            int t0, t1;
            clamp_taps(floorf(src_location(r_lo, ratio_w, off_w, s.roi_x)), x_lo, x_hi, t0, t1);
            x_first = t0;
            clamp_taps(floorf(src_location(r_hi, ratio_w, off_w, s.roi_x)), x_lo, x_hi, t0, t1);
            x_last = t1;
        }

        // Row tables: tap rows, y weights, staging slots.
        const bool dense = !(ratio_h > 2.0f);
        int y_first = 0;
        if (STAGED && dense) {
            int t0, t1;
            clamp_taps(floorf(src_location(s.crop_y + tile_y0, ratio_h, off_h, s.roi_y)), y_lo, y_hi, t0, t1);
            y_first = t0;
        }
        int nslots = 0;
        if (STAGED) {
            if (dense) {
                int t0, t1;
                clamp_taps(floorf(src_location(s.crop_y + tile_y0 + rows_valid - 1, ratio_h, off_h, s.roi_y)), y_lo, y_hi, t0, t1);
                nslots = t1 - y_first + 1;
            } else {
                nslots = 2 * rows_valid;
            }
        }
        if (tid < rows_valid) {
            int ry = s.crop_y + tile_y0 + tid;
            float sy = src_location(ry, ratio_h, off_h, s.roi_y);
            float fy = floorf(sy);
            int y0, y1;
            clamp_taps(fy, y_lo, y_hi, y0, y1);
            RowInfo ri;
            ri.wy = sub_rn(sy, fy);
            ri.owy = sub_rn(1.0f, ri.wy);
            if (STAGED) {
                int s0 = dense ? (y0 - y_first) : 2 * tid;
                int s1 = dense ? (y1 - y_first) : 2 * tid + 1;
                uint32_t m0 = (uint32_t)((uintptr_t)(img + (size_t)y0 * s.src_stride + (size_t)x_first * 3) & 15);
                uint32_t m1 = (uint32_t)((uintptr_t)(img + (size_t)y1 * s.src_stride + (size_t)x_first * 3) & 15);
                ri.off0 = s0 * L.pitch + (int)m0;
                ri.off1 = s1 * L.pitch + (int)m1;
                if (!dense) { srow[2 * tid] = y0; srow[2 * tid + 1] = y1; }
            } else {
                ri.off0 = y0;
                ri.off1 = y1;
            }
            rowinfo[tid] = ri;
        }
        if (STAGED && dense) {
            for (int r = tid; r < nslots; r += TW) srow[r] = y_first + r;
        }
        __syncthreads();

        if (STAGED) {
            const int nbytes = (x_last - x_first + 1) * 3;
            const int cpr = L.pitch >> 4;
            const int total = nslots * cpr;
            for (int idx = tid; idx < total; idx += TW) {
                int r = idx / cpr;
                int ck = idx - r * cpr;
                const uint8_t* g = img + (size_t)srow[r] * s.src_stride + (size_t)x_first * 3;
                uint32_t m = (uint32_t)((uintptr_t)g & 15);
                int need = (int)(m + nbytes + 15) >> 4;
                if (ck < need) cp_async16(stage + (size_t)r * L.pitch + ck * 16, g - m + ck * 16);
            }
            cp_async_commit_wait_all();
            __syncthreads();
        }

        if (tid < cols_valid) {
            int rx = s.crop_x + (s.mirror ? (s.crop_w - 1 - xi) : xi);
            float sx = src_location(rx, ratio_w, off_w, s.roi_x);
            float fx = floorf(sx);
            float wx = sub_rn(sx, fx);
            float owx = sub_rn(1.0f, wx);
            int x0, x1;
            clamp_taps(fx, x_lo, x_hi, x0, x1);
            const int oL = STAGED ? (x0 - x_first) * 3 : x0 * 3;
            const int oR = STAGED ? (x1 - x_first) * 3 : x1 * 3;
            const float mul0 = L.mul[0], mul1 = L.mul[1], mul2 = L.mul[2];
            const float add0 = L.add[0], add1 = L.add[1], add2 = L.add[2];
            for (int j = 0; j < rows_valid; j++) {
                const RowInfo ri = rowinfo[j];
                uint32_t tl, tr, bl, br;
                if (STAGED) {
                    tl = lds_unaligned32(stage, ri.off0 + oL);
                    tr = lds_unaligned32(stage, ri.off0 + oR);
                    bl = lds_unaligned32(stage, ri.off1 + oL);
                    br = lds_unaligned32(stage, ri.off1 + oR);
                } else {
                    const uint8_t* r0 = img + (size_t)ri.off0 * s.src_stride;
                    const uint8_t* r1 = img + (size_t)ri.off1 * s.src_stride;
                    tl = __ldg(r0 + oL) | (__ldg(r0 + oL + 1) << 8) | (__ldg(r0 + oL + 2) << 16);
                    tr = __ldg(r0 + oR) | (__ldg(r0 + oR + 1) << 8) | (__ldg(r0 + oR + 2) << 16);
                    bl = __ldg(r1 + oL) | (__ldg(r1 + oL + 1) << 8) | (__ldg(r1 + oL + 2) << 16);
                    br = __ldg(r1 + oR) | (__ldg(r1 + oR + 1) << 8) | (__ldg(r1 + oR + 2) << 16);
                }
                const float w00 = mul_rn(ri.owy, owx), w01 = mul_rn(ri.owy, wx), w10 = mul_rn(ri.wy, owx);
                float v[3];
#pragma unroll
                for (int c = 0; c < 3; c++) {
                    float ftl = byte_to_float(tl, c), ftr = byte_to_float(tr, c);
                    float fbl = byte_to_float(bl, c), fbr = byte_to_float(br, c);
                    float acc = mul_rn(mul_rn(fbr, ri.wy), wx);
                    acc = fmaf(fbl, w10, acc);
                    acc = fmaf(ftr, w01, acc);
                    acc = fmaf(ftl, w00, acc);
                    v[c] = sat_round_u8f(acc);
                }
                if (L.normalize) {
                    v[0] = fmaf(v[0], mul0, add0);
                    v[1] = fmaf(v[1], mul1, add1);
                    v[2] = fmaf(v[2], mul2, add2);
                }
                store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, tile_y0 + j, xi, v[0], v[1], v[2]);
            }
        }
    }

    if (L.fill_padding && xi < L.out_w) {
        // Zero the part of the tile that lies outside the sample's valid extent.
        const int rows_in_tile = min(L.th, L.out_h - tile_y0);
        for (int j = 0; j < rows_in_tile; j++) {
            int y = tile_y0 + j;
            if (y >= ch || xi >= cw) store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, xi, 0.f, 0.f, 0.f);
        }
    }
}

template <typename OutT, int LAYOUT>
static int launch_typed(const uint8_t* arena, const rb200_resample_sample* samples, int n, const ResampleLaunch& L,
                        int tw, bool staged, size_t smem, cudaStream_t stream) {
    int tiles_y = (L.ext_h + L.th - 1) / L.th;
    dim3 grid((unsigned)(L.tiles_x * tiles_y), (unsigned)n);
    if (staged) {
        auto k = resample_kernel<OutT, LAYOUT, true>;
        if (smem > 48 * 1024) {
            int rc = check_cuda(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                                "cudaFuncSetAttribute(resample)");
            if (rc) return rc;
        }
        k<<<grid, tw, smem, stream>>>(arena, samples, L);
    } else {
        resample_kernel<OutT, LAYOUT, false><<<grid, tw, smem, stream>>>(arena, samples, L);
    }
    RB200_CHECK_LAUNCH("resample_kernel");
    return RB200_OK;
}

}  // namespace rb200

using namespace rb200;

extern "C" int rb200k_resample(const uint8_t* arena, const rb200_resample_sample* samples,
                               const rb200_resample_sample* h_samples, int n, const rb200_resample_params* p,
                               void* stream_v) {
    if (n == 0) return RB200_OK;
    if (!arena || !samples || !p || !p->out || n < 0 || p->out_w <= 0 || p->out_h <= 0) {
        set_error("rb200k_resample: null pointer or non-positive size");
        return RB200_E_INVALID;
    }
    if (n > 65535) {
        set_error("rb200k_resample: batch %d exceeds 65535", n);
        return RB200_E_LIMIT;
    }
    if (p->out_dtype < 0 || p->out_dtype > 2 || (p->out_layout != RB200_NCHW && p->out_layout != RB200_NHWC)) {
        set_error("rb200k_resample: bad out_dtype %d / out_layout %d", p->out_dtype, p->out_layout);
        return RB200_E_INVALID;
    }
    cudaStream_t stream = (cudaStream_t)stream_v;

    ResampleLaunch L;
    L.out = p->out;
    L.out_w = p->out_w;
    L.out_h = p->out_h;
    L.normalize = p->normalize;
    L.fill_padding = p->fill_padding;
    for (int c = 0; c < 3; c++) { L.mul[c] = p->mul[c]; L.add[c] = p->add[c]; }

    // Extent the grid has to cover, and the widest source span a tile can need.
    int ext_w = p->out_w, ext_h = p->out_h;
    if (h_samples) {
        for (int i = 0; i < n; i++) {
            if (h_samples[i].dst_w <= 0 || h_samples[i].dst_h <= 0 || h_samples[i].roi_w <= 0 || h_samples[i].roi_h <= 0) {
                set_error("rb200k_resample: sample %d has an empty roi or target size", i);
                return RB200_E_INVALID;
            }
        }
    }
    if (h_samples && !p->fill_padding) {
        ext_w = 1; ext_h = 1;
        for (int i = 0; i < n; i++) {
            int w = h_samples[i].crop_w < p->out_w ? h_samples[i].crop_w : p->out_w;
            int h = h_samples[i].crop_h < p->out_h ? h_samples[i].crop_h : p->out_h;
            if (w > ext_w) ext_w = w;
            if (h > ext_h) ext_h = h;
        }
    }
    L.ext_w = ext_w;
    L.ext_h = ext_h;
    int tiles_x = (ext_w + 255) / 256;
    int tw = ((ext_w + tiles_x - 1) / tiles_x + 31) & ~31;
    L.tiles_x = (ext_w + tw - 1) / tw;

    bool staged = h_samples != nullptr;
    int pitch = 0, th = 8;
    if (staged) {
        int max_span = 1;
        for (int i = 0; i < n; i++) {
            double ratio = (double)h_samples[i].roi_w / (double)h_samples[i].dst_w;
            long span = (long)(tw * ratio) + 4;
            if (span > h_samples[i].roi_w) span = h_samples[i].roi_w;
            if (span > max_span) max_span = (int)span;
        }
        pitch = (15 + max_span * 3 + 8 + 15) & ~15;
        const size_t budget = 40 * 1024, hard = 160 * 1024;
        th = 8;
        while (th > 1 && (size_t)(2 * th + 2) * pitch > budget) th >>= 1;
        if ((size_t)(2 * th + 2) * pitch > hard) staged = false;
    }
    if (!staged) { pitch = 0; th = 8; }
    L.th = th;
    L.pitch = pitch;
    size_t smem = ((sizeof(RowInfo) * th + sizeof(int) * (2 * th + 2) + 15) & ~(size_t)15) +
                  (staged ? (size_t)(2 * th + 2) * pitch : 0);

#define RB200_DISPATCH(T, LAY) return launch_typed<T, LAY>(arena, samples, n, L, tw, staged, smem, stream)
    if (p->out_layout == RB200_NCHW) {
        if (p->out_dtype == RB200_FP32) RB200_DISPATCH(float, RB200_NCHW);
        if (p->out_dtype == RB200_FP16) RB200_DISPATCH(__half, RB200_NCHW);
        RB200_DISPATCH(uint8_t, RB200_NCHW);
    } else {
        if (p->out_dtype == RB200_FP32) RB200_DISPATCH(float, RB200_NHWC);
        if (p->out_dtype == RB200_FP16) RB200_DISPATCH(__half, RB200_NHWC);
        RB200_DISPATCH(uint8_t, RB200_NHWC);
    }
#undef RB200_DISPATCH
}
