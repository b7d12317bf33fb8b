// Pointwise family: window (crop) + flips + colour arithmetic + per-channel fma + layout/dtype
// conversion, one launch for the whole batch. grid = (tiles of the output extent, samples).
//
// Colour arithmetic is float32 on the 0..255 scale with one rounding per operation:
//   brightness  y = alpha*x + beta
//   contrast    y = (x - center)*factor + center
//   twist       hexcone RGB->HSV, H += hue (wrapped to [0,360)), S = clamp(S*sat,0,1), HSV->RGB,
//               then alpha*x + beta
// The colour result is rounded to nearest even and saturated to uint8 before the optional
// normalisation (the reference's colour nodes output uint8 tensors).
#include "common.cuh"

namespace rb200 {

struct PointwiseLaunch {
    void* out;
    int out_w, out_h;
    int ext_w, ext_h;
    int tiles_x;
    int th;
    int color_op, normalize, fill_padding, reverse_channels;
    float mul[3], add[3];
};

__device__ __forceinline__ void color_twist_px(float r, float g, float b, float hue, float sat, float& o0, float& o1, float& o2) {
    float cmax = fmaxf(r, fmaxf(g, b));
    float cmin = fminf(r, fminf(g, b));
    float delta = sub_rn(cmax, cmin);
    float h = 0.f, s = 0.f, v = cmax;
    if (delta > 0.f) {
        s = div_rn(delta, cmax);
        if (cmax == r) {
            h = mul_rn(60.f, div_rn(sub_rn(g, b), delta));
            if (h < 0.f) h = add_rn(h, 360.f);
        } else if (cmax == g) {
            h = add_rn(mul_rn(60.f, div_rn(sub_rn(b, r), delta)), 120.f);
        } else {
            h = add_rn(mul_rn(60.f, div_rn(sub_rn(r, g), delta)), 240.f);
        }
    }
    h = add_rn(h, hue);
    h = sub_rn(h, mul_rn(360.f, floorf(mul_rn(h, 1.0f / 360.f))));
    s = mul_rn(s, sat);
    s = fminf(fmaxf(s, 0.f), 1.f);
    float hp = mul_rn(h, 1.0f / 60.f);
    float fi = floorf(hp);
    float f = sub_rn(hp, fi);
    int sector = (int)fi;
    if (sector >= 6) sector -= 6;
    if (sector < 0) sector = 0;
    float pp = mul_rn(v, sub_rn(1.f, s));
    float qq = mul_rn(v, sub_rn(1.f, mul_rn(s, f)));
    float tt = mul_rn(v, sub_rn(1.f, mul_rn(s, sub_rn(1.f, f))));
    switch (sector) {
        case 0: o0 = v; o1 = tt; o2 = pp; break;
        case 1: o0 = qq; o1 = v; o2 = pp; break;
        case 2: o0 = pp; o1 = v; o2 = tt; break;
        case 3: o0 = pp; o1 = qq; o2 = v; break;
        case 4: o0 = tt; o1 = pp; o2 = v; break;
        default: o0 = v; o1 = pp; o2 = qq; break;
    }
}

template <typename OutT, int LAYOUT>
__device__ __forceinline__ void pw_store3(OutT* out, int out_w, int out_h, int n, int y, int x, float v0, float v1, float v2) {
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

template <typename OutT, int LAYOUT, int COLOR_OP>
__global__ void __launch_bounds__(256) pointwise_kernel(const uint8_t* __restrict__ arena,
                                                        const rb200_pointwise_sample* __restrict__ samples,
                                                        const PointwiseLaunch L) {
    const int n = blockIdx.y;
    const int tx = blockIdx.x % L.tiles_x;
    const int ty = blockIdx.x / L.tiles_x;
    const int xi = tx * blockDim.x + threadIdx.x;
    const int tile_y0 = ty * L.th;

    const rb200_pointwise_sample s = samples[n];
    const uint8_t* img = arena + s.src_offset;
    OutT* out = reinterpret_cast<OutT*>(L.out);
    const int w = min(s.roi_w, L.out_w);
    const int h = min(s.roi_h, L.out_h);

    if (xi < w) {
        const int sx = s.roi_x + (s.flip_h ? (s.roi_w - 1 - xi) : xi);
        const int rows = min(L.th, h - tile_y0);
        for (int j = 0; j < rows; j++) {
            const int y = tile_y0 + j;
            const int sy = s.roi_y + (s.flip_v ? (s.roi_h - 1 - y) : y);
            const uint8_t* px = img + (size_t)sy * s.src_stride + (size_t)sx * 3;
            float p0 = (float)__ldg(px), p1 = (float)__ldg(px + 1), p2 = (float)__ldg(px + 2);
            float v0, v1, v2;
            if (COLOR_OP == RB200_COLOR_BRIGHTNESS) {
                v0 = sat_round_u8f(add_rn(mul_rn(s.alpha, p0), s.beta));
                v1 = sat_round_u8f(add_rn(mul_rn(s.alpha, p1), s.beta));
                v2 = sat_round_u8f(add_rn(mul_rn(s.alpha, p2), s.beta));
            } else if (COLOR_OP == RB200_COLOR_CONTRAST) {
                v0 = sat_round_u8f(add_rn(mul_rn(sub_rn(p0, s.beta), s.alpha), s.beta));
                v1 = sat_round_u8f(add_rn(mul_rn(sub_rn(p1, s.beta), s.alpha), s.beta));
                v2 = sat_round_u8f(add_rn(mul_rn(sub_rn(p2, s.beta), s.alpha), s.beta));
            } else if (COLOR_OP == RB200_COLOR_TWIST) {
                float t0, t1, t2;
                color_twist_px(p0, p1, p2, s.hue, s.sat, t0, t1, t2);
                v0 = sat_round_u8f(add_rn(mul_rn(s.alpha, t0), s.beta));
                v1 = sat_round_u8f(add_rn(mul_rn(s.alpha, t1), s.beta));
                v2 = sat_round_u8f(add_rn(mul_rn(s.alpha, t2), s.beta));
            } else {
                v0 = p0; v1 = p1; v2 = p2;
            }
            if (L.reverse_channels) { float t = v0; v0 = v2; v2 = t; }
            if (L.normalize) {
                v0 = fmaf(v0, L.mul[0], L.add[0]);
                v1 = fmaf(v1, L.mul[1], L.add[1]);
                v2 = fmaf(v2, L.mul[2], L.add[2]);
            }
            pw_store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, xi, v0, v1, v2);
        }
    }
    if (L.fill_padding && xi < L.out_w) {
        const int rows_in_tile = min(L.th, L.out_h - tile_y0);
        for (int j = 0; j < rows_in_tile; j++) {
            int y = tile_y0 + j;
            if (y >= h || xi >= w) pw_store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, xi, 0.f, 0.f, 0.f);
        }
    }
}

template <typename OutT, int LAYOUT>
static int launch_color(int color_op, dim3 grid, int tw, cudaStream_t stream, const uint8_t* arena,
                        const rb200_pointwise_sample* samples, const PointwiseLaunch& L) {
    switch (color_op) {
        case RB200_COLOR_NONE: pointwise_kernel<OutT, LAYOUT, RB200_COLOR_NONE><<<grid, tw, 0, stream>>>(arena, samples, L); break;
        case RB200_COLOR_BRIGHTNESS: pointwise_kernel<OutT, LAYOUT, RB200_COLOR_BRIGHTNESS><<<grid, tw, 0, stream>>>(arena, samples, L); break;
        case RB200_COLOR_CONTRAST: pointwise_kernel<OutT, LAYOUT, RB200_COLOR_CONTRAST><<<grid, tw, 0, stream>>>(arena, samples, L); break;
        case RB200_COLOR_TWIST: pointwise_kernel<OutT, LAYOUT, RB200_COLOR_TWIST><<<grid, tw, 0, stream>>>(arena, samples, L); break;
        default: set_error("rb200k_pointwise: bad color_op %d", color_op); return RB200_E_INVALID;
    }
    RB200_CHECK_LAUNCH("pointwise_kernel");
    return RB200_OK;
}

}  // namespace rb200

using namespace rb200;

extern "C" int rb200k_pointwise(const uint8_t* arena, const rb200_pointwise_sample* samples,
                                const rb200_pointwise_sample* h_samples, int n, const rb200_pointwise_params* p,
                                void* stream_v) {
    if (n == 0) return RB200_OK;
    if (!arena || !samples || !p || !p->out || n < 0 || p->out_w <= 0 || p->out_h <= 0) {
        set_error("rb200k_pointwise: null pointer or non-positive size");
        return RB200_E_INVALID;
    }
    if (n > 65535) {
        set_error("rb200k_pointwise: batch %d exceeds 65535", n);
        return RB200_E_LIMIT;
    }
    if (p->out_dtype < 0 || p->out_dtype > 2 || (p->out_layout != RB200_NCHW && p->out_layout != RB200_NHWC)) {
        set_error("rb200k_pointwise: bad out_dtype %d / out_layout %d", p->out_dtype, p->out_layout);
        return RB200_E_INVALID;
    }
    cudaStream_t stream = (cudaStream_t)stream_v;
    PointwiseLaunch L;
    L.out = p->out;
    L.out_w = p->out_w;
    L.out_h = p->out_h;
    L.color_op = p->color_op;
    L.normalize = p->normalize;
    L.fill_padding = p->fill_padding;
    L.reverse_channels = p->reverse_channels;
    for (int c = 0; c < 3; c++) { L.mul[c] = p->mul[c]; L.add[c] = p->add[c]; }
    int ext_w = p->out_w, ext_h = p->out_h;
    if (h_samples && !p->fill_padding) {
        ext_w = 1; ext_h = 1;
        for (int i = 0; i < n; i++) {
            int w = h_samples[i].roi_w < p->out_w ? h_samples[i].roi_w : p->out_w;
            int h = h_samples[i].roi_h < p->out_h ? h_samples[i].roi_h : p->out_h;
            if (w > ext_w) ext_w = w;
            if (h > ext_h) ext_h = h;
        }
    }
    L.ext_w = ext_w;
    L.ext_h = ext_h;
    int tiles_x = (ext_w + 255) / 256;
    int tw = ((ext_w + tiles_x - 1) / tiles_x + 31) & ~31;
    L.tiles_x = (ext_w + tw - 1) / tw;
    L.th = 8;
    int tiles_y = (ext_h + L.th - 1) / L.th;
    dim3 grid((unsigned)(L.tiles_x * tiles_y), (unsigned)n);

#define RB200_DISPATCH(T, LAY) return launch_color<T, LAY>(p->color_op, grid, tw, stream, arena, samples, L)
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
