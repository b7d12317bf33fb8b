/*
 * oracle.c — CPU restatement of the rocAL augmentation hot path. TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA kernels are compared with. It is never part of the
 * product path: only the tests, the smoke check and the benchmark's CPU-baseline leg load it.
 *
 * Parity status
 *   - orc_box_encode, orc_box_iou_match: PINNED against the reference's own BoundingBoxGraph compiled from the
 *     reference sources (ref_driver.cpp) and against golden vectors generated from that build.
 *   - orc_resample with bilinear or triangular interpolation on a whole-image ROI, and the x*mul+add
 *     conversion of orc_pointwise: PINNED against the reference's own pixel kernels — the in-tree HIP kernels
 *     resize_bilinear_pkd_hip_tensor, resize_generic_pln1_hip_tensor and Hip_CopyInt8To* of
 *     rocAL/rocAL_hip/rocal_hip_kernels.cpp compiled for the host (ref_hip_driver.cpp, ref_stubs/hip/) — bit
 *     for bit, on golden vectors from that build and on the live build where the reference tree exists.
 *     Products that feed a sum inside one expression of those kernels are fused multiply-adds, as the HIP
 *     compiler builds them; they are spelled fmaf() here.
 *   - orc_crop_fixed: PINNED against RocalCropParam::fill_crop_dims compiled in place.
 *   - Everything else in orc_resample / orc_pointwise / orc_warp_affine (crop windows and mirrors applied to the
 *     resize, the normalisation of CropMirrorNormalize, the colour operators, the affine gather, the other
 *     filters): PARITY UNPINNED. The reference executes these operators inside the RPP library through
 *     MIVisionX/OpenVX; neither is present in the reference tree, and the reference's golden images live in
 *     an external data tree. The arithmetic follows the pinned kernels where they apply (the bilinear tap rule
 *     and packing) and the node / meta-node / API files cited at each function.
 *
 * All float arithmetic is IEEE binary32 with one rounding per written operation (build with
 * -ffp-contract=off); fused multiply-adds are spelled fmaf().
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/rb200_kernels.h"

#define ORC_API __attribute__((visibility("default")))

static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* Round to nearest even and saturate to [0,255]: the packing step of the HIP kernels
 * (cvt_pk_u8_f32, rocAL/rocAL_hip/rocal_hip_kernels.cpp:425-430). */
static inline uint8_t sat_u8(float v) {
    float r = nearbyintf(v);
    if (!(r > 0.f)) return 0; /* also NaN */
    if (r > 255.f) return 255;
    return (uint8_t)r;
}

static inline uint16_t f32_to_f16_bits(float f) {
    _Float16 h = (_Float16)f; /* round to nearest even, as __float2half (rocal_hip_kernels.cpp:119-121) */
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

static inline void store_elem(void* out, int dtype, size_t idx, float v) {
    if (dtype == RB200_FP32)
        ((float*)out)[idx] = v;
    else if (dtype == RB200_FP16)
        ((uint16_t*)out)[idx] = f32_to_f16_bits(v);
    else
        ((uint8_t*)out)[idx] = sat_u8(v);
}

static inline size_t out_index(int layout, int out_w, int out_h, int n, int c, int y, int x) {
    if (layout == RB200_NCHW) return (((size_t)n * 3 + c) * out_h + y) * out_w + x;
    return (((size_t)n * out_h + y) * out_w + x) * 3 + c;
}

static void fill_sample_zero(void* out, int dtype, int out_w, int out_h, int n) {
    size_t elems = (size_t)3 * out_w * out_h;
    size_t esz = dtype == RB200_FP32 ? 4 : (dtype == RB200_FP16 ? 2 : 1);
    memset((uint8_t*)out + (size_t)n * elems * esz, 0, elems * esz);
}

/* ------------------------------------------------------------------------------------------
 * Bilinear sample of one source position, 3 channels.
 * Follows rocAL/rocAL_hip/rocal_hip_kernels.cpp:
 *   :388-409  floor, weights = frac / 1-frac, optional range check -> 0
 *   :340-343  both taps clamped to [roi.x, roi.z-1] x [roi.y, roi.w-1], roi.z/.w being the
 *             inclusive right/bottom coordinate (:469-472)
 *   :332-337  fmaf nesting  TL*(1-wy)(1-wx) + (TR*(1-wy)wx + (BL*wy(1-wx) + BR*wy*wx))
 * The upper clamp bound is kept >= the lower one so that 1-pixel-wide sources stay in range.
 * ---------------------------------------------------------------------------------------- */
static inline int bilinear3(const uint8_t* img, uint32_t stride, int x_lo, int y_lo, int x_hi_incl,
                            int y_hi_incl, float sx, float sy, int check_range, float out[3]) {
    float fx = floorf(sx), fy = floorf(sy);
    if (check_range && (fx < (float)x_lo || fy < (float)y_lo || fx > (float)x_hi_incl || fy > (float)y_hi_incl)) {
        out[0] = out[1] = out[2] = 0.f;
        return 0;
    }
    float wx = sx - fx, wy = sy - fy;
    float owx = 1.0f - wx, owy = 1.0f - wy;
    int cx_hi = x_hi_incl - 1 > x_lo ? x_hi_incl - 1 : x_lo;
    int cy_hi = y_hi_incl - 1 > y_lo ? y_hi_incl - 1 : y_lo;
    int x0 = (int)fminf(fmaxf(fx, (float)x_lo), (float)cx_hi);
    int y0 = (int)fminf(fmaxf(fy, (float)y_lo), (float)cy_hi);
    int x1 = (int)fminf(fmaxf(fx + 1.0f, (float)x_lo), (float)cx_hi);
    int y1 = (int)fminf(fmaxf(fy + 1.0f, (float)y_lo), (float)cy_hi);
    const uint8_t* r0 = img + (size_t)y0 * stride;
    const uint8_t* r1 = img + (size_t)y1 * stride;
    float w00 = owy * owx, w01 = owy * wx, w10 = wy * owx;
    for (int c = 0; c < 3; c++) {
        float tl = (float)r0[x0 * 3 + c], tr = (float)r0[x1 * 3 + c];
        float bl = (float)r1[x0 * 3 + c], br = (float)r1[x1 * 3 + c];
        out[c] = fmaf(tl, w00, fmaf(tr, w01, fmaf(bl, w10, br * wy * wx)));
    }
    return 1;
}

/* ------------------------------------------------------------------------------------------
 * Triangular ("generic") resize of one output position, 3 channels. Follows
 * resize_generic_pln1_hip_tensor and its helpers (rocAL/rocAL_hip/rocal_hip_kernels.cpp):
 *   :508-513  ratio > 1: radius = ratio, scale = 1/ratio; else radius = scale = 1
 *   :553-556  offset = (ratio-1)/2 - radius, kernel size = ceil(2*radius)
 *   :487-492  first tap = ceil(dst*ratio + offset + roi), weight = first - raw, first clamped from
 *             above to the last source index
 *   :494-497  coefficient = max(0, 1 - |(weight - radius + j) * scale|)
 *   :567-580  rows outer, columns inner, taps clamped to the source, out += src * (col*row)
 *   :582-587  out *= 1 / (row_sum * col_sum) (a zero sum counts as 1), clamp to [0,255], truncate.
 * The in-tree kernel handles one channel; here it runs on each of the three interleaved channels, and
 * the clamp range is the sample's ROI. Products feeding the running sum are one fmaf each.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
    float radius, scale, offset;
    int ksize;
} tri_axis;

static inline tri_axis tri_axis_make(float ratio) {
    tri_axis a;
    if (ratio > 1.0f) { a.radius = ratio; a.scale = 1.0f / ratio; } else { a.radius = 1.0f; a.scale = 1.0f; }
    a.offset = (ratio - 1.0f) * 0.5f - a.radius;
    a.ksize = (int)ceilf(a.radius * 2.0f);
    return a;
}

static inline void tri_loc(const tri_axis* a, float ratio, int dst, int roi_lo, int limit, int* first, float* weight) {
    float raw = fmaf((float)dst, ratio, a->offset) + (float)roi_lo;
    int r = (int)ceilf(raw);
    *weight = (float)r - raw;
    *first = r > limit ? limit : r;
}

static inline float tri_coeff(const tri_axis* a, float weight, int j) {
    float c = 1.0f - fabsf(((weight - a->radius) + (float)j) * a->scale);
    return c < 0.f ? 0.f : c;
}

/* The other filters of the resize family on the same skeleton. The reference names them
 * (rocAL/include/api/rocal_api_types.h:347-367) but their arithmetic lives in RPP, so these
 * definitions are this library's own: base radius B per filter, radius = B * max(ratio, 1),
 * scale = 1 / max(ratio, 1), the weight function evaluated at (weight - radius + j) * scale. */
static inline float filter_base_radius(int filter) {
    switch (filter) {
        case RB200_INTERP_BICUBIC: return 2.0f;
        case RB200_INTERP_LANCZOS: return 3.0f;
        case RB200_INTERP_NEAREST: return 0.5f;
        default: return 1.0f;   /* triangular, gaussian */
    }
}

static inline tri_axis filter_axis_make(float ratio, int filter) {
    if (filter == RB200_INTERP_TRIANGULAR) return tri_axis_make(ratio);
    tri_axis a;
    const float stretch = ratio > 1.0f ? ratio : 1.0f;
    a.radius = filter_base_radius(filter) * stretch;
    a.scale = ratio > 1.0f ? 1.0f / ratio : 1.0f;
    a.offset = (ratio - 1.0f) * 0.5f - a.radius;
    a.ksize = (int)ceilf(a.radius * 2.0f);
    if (a.ksize < 1) a.ksize = 1;
    return a;
}

static inline float filter_weight(int filter, float x) {
    const float ax = fabsf(x);
    switch (filter) {
        case RB200_INTERP_BICUBIC:   /* Keys, a = -0.5 */
            if (ax >= 2.0f) return 0.f;
            if (ax > 1.0f) return fmaf(-4.0f, ax, (ax * ax) * fmaf(-0.5f, ax, 2.5f)) + 2.0f;
            return fmaf(ax * ax, fmaf(1.5f, ax, -2.5f), 1.0f);
        case RB200_INTERP_LANCZOS: {
            if (ax >= 3.0f) return 0.f;
            if (ax < 1e-5f) return 1.0f;
            const float px = ax * 3.14159265358979323846f;
            return (3.0f * (sinf(px) * sinf(px * (1.0f / 3.0f)))) / (px * px);
        }
        case RB200_INTERP_GAUSSIAN: return expf(-4.0f * (x * x));
        case RB200_INTERP_NEAREST: return 1.0f;
        default: {
            const float c = 1.0f - ax;
            return c < 0.f ? 0.f : c;
        }
    }
}

static inline float filter_coeff(const tri_axis* a, int filter, float weight, int j) {
    if (filter == RB200_INTERP_TRIANGULAR) return tri_coeff(a, weight, j);
    return filter_weight(filter, ((weight - a->radius) + (float)j) * a->scale);
}


static inline uint8_t trunc_u8(float v) {
    v = fmaxf(fminf(v, 255.f), 0.f);   /* NaN -> 0 through fmaxf */
    return (uint8_t)v;
}

static void triangular3(const uint8_t* img, uint32_t stride, int x_lo, int y_lo, int x_hi, int y_hi,
                        const tri_axis* ax, const tri_axis* ay, float ratio_w, float ratio_h, int dx, int dy,
                        int filter, uint8_t out[3]) {
    int fx, fy;
    float wx, wy;
    tri_loc(ax, ratio_w, dx, x_lo, x_hi, &fx, &wx);
    tri_loc(ay, ratio_h, dy, y_lo, y_hi, &fy, &wy);
    float acc[3] = {0.f, 0.f, 0.f};
    float row_sum = 0.f, col_sum = 0.f;
    for (int j = 0; j < ay->ksize; j++) {
        int row = clampi(fy + j, y_lo, y_hi);
        const uint8_t* r = img + (size_t)row * stride;
        float rc = filter_coeff(ay, filter, wy, j);
        row_sum += rc;
        col_sum = 0.f;
        for (int k = 0; k < ax->ksize; k++) {
            int col = clampi(fx + k, x_lo, x_hi);
            float cc = filter_coeff(ax, filter, wx, k);
            col_sum += cc;
            float coeff = cc * rc;
            for (int c = 0; c < 3; c++) acc[c] = fmaf((float)r[col * 3 + c], coeff, acc[c]);
        }
    }
    if (row_sum == 0.f) row_sum = 1.f;
    if (col_sum == 0.f) col_sum = 1.f;
    float inv = 1.0f / (row_sum * col_sum);
    for (int c = 0; c < 3; c++) out[c] = trunc_u8(acc[c] * inv);
}

/* ------------------------------------------------------------------------------------------
 * Resample family. Per sample: resize the source rectangle roi to dst_w x dst_h (bilinear),
 * quantise to uint8 (the reference's Resize node outputs uint8 before the next node reads
 * it), take the window crop_*, mirror, then either store the uint8 or fma(u8, mul, add).
 *   source location: dst*ratio + (ratio-1)/2 + roi.x, ratio = roi_dim/dst_dim
 *                    (rocal_hip_kernels.cpp:311-329)
 *   crop+mirror+normalize: out = (src - mean)/std evaluated as x*(1/std) + (-mean*(1/std)),
 *                    the two tables the node builds (node_crop_mirror_normalize.cpp:46-70)
 * ---------------------------------------------------------------------------------------- */
ORC_API int orc_resample(const uint8_t* arena, const rb200_resample_sample* s, int n,
                         const rb200_resample_params* p) {
    if (!arena || !s || !p || !p->out || n < 0) return RB200_E_INVALID;
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < n; i++) {
        const rb200_resample_sample* q = &s[i];
        const uint8_t* img = arena + q->src_offset;
        if (p->fill_padding) fill_sample_zero(p->out, p->out_dtype, p->out_w, p->out_h, i);
        float ratio_w = (float)q->roi_w / (float)q->dst_w;
        float ratio_h = (float)q->roi_h / (float)q->dst_h;
        float off_w = (ratio_w - 1.0f) * 0.5f;
        float off_h = (ratio_h - 1.0f) * 0.5f;
        int x_hi = q->roi_x + q->roi_w - 1, y_hi = q->roi_y + q->roi_h - 1;
        int cw = q->crop_w < p->out_w ? q->crop_w : p->out_w;
        int ch = q->crop_h < p->out_h ? q->crop_h : p->out_h;
        const int generic = p->interpolation != RB200_INTERP_BILINEAR;
        tri_axis ax = filter_axis_make(ratio_w, p->interpolation), ay = filter_axis_make(ratio_h, p->interpolation);
        for (int y = 0; y < ch; y++) {
            int ry = q->crop_y + y;
            float sy = fmaf((float)ry, ratio_h, off_h) + (float)q->roi_y;
            for (int x = 0; x < cw; x++) {
                int rx = q->crop_x + (q->mirror ? (q->crop_w - 1 - x) : x);
                float sx = fmaf((float)rx, ratio_w, off_w) + (float)q->roi_x;
                float v[3] = {0.f, 0.f, 0.f};
                uint8_t t3[3] = {0, 0, 0};
                if (generic)
                    triangular3(img, q->src_stride, q->roi_x, q->roi_y, x_hi, y_hi, &ax, &ay, ratio_w, ratio_h, rx, ry,
                                p->interpolation, t3);
                else
                    bilinear3(img, q->src_stride, q->roi_x, q->roi_y, x_hi, y_hi, sx, sy, 0, v);
                for (int c = 0; c < 3; c++) {
                    float u = generic ? (float)t3[c] : (float)sat_u8(v[c]);
                    float o = p->normalize ? fmaf(u, p->mul[c], p->add[c]) : u;
                    store_elem(p->out, p->out_dtype, out_index(p->out_layout, p->out_w, p->out_h, i, c, y, x), o);
                }
            }
        }
    }
    return RB200_OK;
}

/* ------------------------------------------------------------------------------------------
 * Colour arithmetic (float32 on the 0..255 scale).
 *   brightness: y = alpha*x + beta              (rocAL/include/api/rocal_api_augmentation.h:226-236)
 *   contrast  : y = (x - center)*factor + center (rocal_api_augmentation.h:290-301)
 *   twist     : RGB -> HSV (H in degrees, S in [0,1], V on the 0..255 scale), H += hue (wrapped
 *               to [0,360)), S = clamp(S*sat, 0, 1), HSV -> RGB, then y = alpha*x + beta
 *               (parameter meaning: rocal_api_augmentation.h:866-877). The reference holds no
 *               arithmetic for this operator (it runs in RPP): the formula is this
 *               restatement's own, the textbook hexcone model, written with reciprocal
 *               multiplies (S = delta * (1/max), H = 60 * (num * (1/delta)) + offset) and the
 *               branch-free inverse  channel = V - V*S*clamp(min(k, 4-k), 0, 1).
 * ---------------------------------------------------------------------------------------- */
static inline float hsv_channel(float v, float vs, float hp, float nshift) {
    float k = nshift + hp;
    if (k >= 6.f) k = k - 6.f;
    float t = fminf(k, 4.f - k);
    t = fminf(fmaxf(t, 0.f), 1.f);
    return v - vs * t;
}

static inline void color_twist_px(float r, float g, float b, float hue, float sat, float out[3]) {
    float cmax = fmaxf(r, fmaxf(g, b));
    float cmin = fminf(r, fminf(g, b));
    float delta = cmax - cmin;
    /* reciprocals of the (integer valued) range and maximum; 0 stands in for 1/0 so that grey pixels
     * get hue 0 and saturation 0 */
    float rd = delta > 0.f ? 1.0f / delta : 0.f;
    float rm = cmax > 0.f ? 1.0f / cmax : 0.f;
    float s = delta * rm;
    float num, offs;
    if (cmax == r) { num = g - b; offs = 0.f; }
    else if (cmax == g) { num = b - r; offs = 120.f; }
    else { num = r - g; offs = 240.f; }
    float h = 60.f * (num * rd) + offs;
    if (h < 0.f) h = h + 360.f;
    float v = cmax;
    h = h + hue;
    h = h - 360.f * floorf(h * (1.0f / 360.f));
    s = s * sat;
    s = fminf(fmaxf(s, 0.f), 1.f);
    float hp = h * (1.0f / 60.f);
    float vs = v * s;
    /* HSV -> RGB: channel = V - V*S*clamp(min(k, 4-k), 0, 1), k = (n + H/60) mod 6, n = 5, 3, 1 */
    out[0] = hsv_channel(v, vs, hp, 5.f);
    out[1] = hsv_channel(v, vs, hp, 3.f);
    out[2] = hsv_channel(v, vs, hp, 1.f);
}

/* Pointwise family: window + flips (pure indexing; vxExtRppCrop / vxExtRppFlip semantics of
 * node_crop.cpp:101-119 and node_flip.cpp:31-64, bbox twin in meta_node_flip.cpp:40-55),
 * colour op, uint8 quantisation of the colour result, optional per-channel fma and channel
 * reversal (x*mult+off of rocal_hip_kernels.cpp:40-217 / master_graph.cpp:672-853). */
ORC_API int orc_pointwise(const uint8_t* arena, const rb200_pointwise_sample* s, int n,
                          const rb200_pointwise_params* p) {
    if (!arena || !s || !p || !p->out || n < 0) return RB200_E_INVALID;
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < n; i++) {
        const rb200_pointwise_sample* q = &s[i];
        const uint8_t* img = arena + q->src_offset;
        if (p->fill_padding) fill_sample_zero(p->out, p->out_dtype, p->out_w, p->out_h, i);
        int w = q->roi_w < p->out_w ? q->roi_w : p->out_w;
        int h = q->roi_h < p->out_h ? q->roi_h : p->out_h;
        for (int y = 0; y < h; y++) {
            int sy = q->roi_y + (q->flip_v ? (q->roi_h - 1 - y) : y);
            const uint8_t* row = img + (size_t)sy * q->src_stride;
            for (int x = 0; x < w; x++) {
                int sx = q->roi_x + (q->flip_h ? (q->roi_w - 1 - x) : x);
                float px[3] = {(float)row[sx * 3], (float)row[sx * 3 + 1], (float)row[sx * 3 + 2]};
                float v[3];
                switch (p->color_op) {
                    case RB200_COLOR_BRIGHTNESS: {   /* hue tilts the offset: exposure / colour temperature are this case */
                        const float bc[3] = {q->beta + q->hue, q->beta, q->beta - q->hue};
                        for (int c = 0; c < 3; c++) v[c] = (float)sat_u8(q->alpha * px[c] + bc[c]);
                        break;
                    }
                    case RB200_COLOR_BLEND: {
                        const uint8_t* img2 = arena + (((uint64_t)q->src2_offset_hi << 32) | q->src2_offset_lo);
                        const uint8_t* p2 = img2 + (size_t)sy * q->src2_stride + (size_t)sx * 3;
                        const float w2 = 1.0f - q->alpha;
                        for (int c = 0; c < 3; c++) v[c] = (float)sat_u8(q->alpha * px[c] + w2 * (float)p2[c]);
                        break;
                    }
                    case RB200_COLOR_GAMMA:
                        for (int c = 0; c < 3; c++) v[c] = (float)sat_u8(255.0f * powf(px[c] * (1.0f / 255.0f), q->alpha));
                        break;
                    case RB200_COLOR_CONTRAST:
                        for (int c = 0; c < 3; c++) v[c] = (float)sat_u8((px[c] - q->beta) * q->alpha + q->beta);
                        break;
                    case RB200_COLOR_TWIST: {
                        float t[3];
                        color_twist_px(px[0], px[1], px[2], q->hue, q->sat, t);
                        for (int c = 0; c < 3; c++) v[c] = (float)sat_u8(q->alpha * t[c] + q->beta);
                        break;
                    }
                    default:
                        v[0] = px[0]; v[1] = px[1]; v[2] = px[2];
                }
                for (int c = 0; c < 3; c++) {
                    int sc = p->reverse_channels ? 2 - c : c;
                    float o = p->normalize ? fmaf(v[sc], p->mul[c], p->add[c]) : v[sc];
                    store_elem(p->out, p->out_dtype, out_index(p->out_layout, p->out_w, p->out_h, i, c, y, x), o);
                }
            }
        }
    }
    return RB200_OK;
}

/* ------------------------------------------------------------------------------------------
 * Affine gather. Table packing [m00, m01, m10, m11, t0, t1] = [x0, y0, x1, y1, o0, o1]
 * (node_warp_affine.cpp:43-48). Centres: output coordinates relative to the integer half of
 * the output size, source coordinates relative to half the source size in float — the
 * centres the rotate bbox twin uses (meta_data/meta_node_rotate.cpp:60-64). Positions whose
 * floor lies outside the source give 0 (the range-check branch, rocal_hip_kernels.cpp:396-398).
 * ---------------------------------------------------------------------------------------- */
ORC_API int orc_warp_affine(const uint8_t* arena, const rb200_warp_sample* s, int n,
                            const rb200_warp_params* p) {
    if (!arena || !s || !p || !p->out || n < 0) return RB200_E_INVALID;
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < n; i++) {
        const rb200_warp_sample* q = &s[i];
        const uint8_t* img = arena + q->src_offset;
        if (p->fill_padding) fill_sample_zero(p->out, RB200_UINT8, p->out_w, p->out_h, i);
        int w = q->dst_w < p->out_w ? q->dst_w : p->out_w;
        int h = q->dst_h < p->out_h ? q->dst_h : p->out_h;
        float cx = (float)(q->dst_w / 2), cy = (float)(q->dst_h / 2);
        float t0 = q->m[4] + (float)q->src_w * 0.5f;
        float t1 = q->m[5] + (float)q->src_h * 0.5f;
        uint8_t* out = (uint8_t*)p->out + (size_t)i * p->out_w * p->out_h * 3;
        for (int y = 0; y < h; y++) {
            float dy = (float)y - cy;
            for (int x = 0; x < w; x++) {
                float dx = (float)x - cx;
                float sx = fmaf(q->m[0], dx, fmaf(q->m[1], dy, t0));
                float sy = fmaf(q->m[2], dx, fmaf(q->m[3], dy, t1));
                float v[3];
                bilinear3(img, q->src_stride, 0, 0, q->src_w - 1, q->src_h - 1, sx, sy, 1, v);
                for (int c = 0; c < 3; c++) out[((size_t)y * p->out_w + x) * 3 + c] = sat_u8(v[c]);
            }
        }
    }
    return RB200_OK;
}

/* ------------------------------------------------------------------------------------------
 * SSD box encoder. Restates BoundingBoxGraph::update_box_encoder_meta_data
 * (rocAL/source/meta_data/bounding_box_graph.cpp:150-220) with its helpers:
 *   :61-69    IoU = inter / (area1 + area2 - inter)
 *   :120-136  per box: IoU against every anchor; best anchor by strict '>' (lowest index
 *             among equals) gets IoU 2.0
 *   :138-148  per anchor: best box by '>=' (highest index among equals)
 *   :173-216  match if IoU > criteria; offset encoding or plain xcycwh; unmatched anchors
 *             give label 0 and zeros (offset) or the anchor as xcycwh.
 * All pointers are host pointers.
 * ---------------------------------------------------------------------------------------- */
static inline float iou_ltrb(const float* b1, float area1, const float* b2) {
    float xa = fmaxf(b1[0], b2[0]), ya = fmaxf(b1[1], b2[1]);
    float xb = fminf(b1[2], b2[2]), yb = fminf(b1[3], b2[3]);
    float inter = fmaxf(0.f, xb - xa) * fmaxf(0.f, yb - ya);
    float area2 = (b2[3] - b2[1]) * (b2[2] - b2[0]);
    return inter / (area1 + area2 - inter);
}

ORC_API int orc_box_encode(const float* boxes, const int32_t* labels, const int32_t* box_offsets, int n,
                           const float* anchors, int num_anchors, float criteria, const float* means,
                           const float* stds, int offset, float scale, float* out_boxes,
                           int32_t* out_labels) {
    if (!boxes || !labels || !box_offsets || !anchors || !out_boxes || !out_labels) return RB200_E_INVALID;
    float inv_stds[4];
    for (int k = 0; k < 4; k++) inv_stds[k] = (float)(1. / stds[k]);
    float half_scale = (float)(0.5 * scale);
    int A = num_anchors;
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < n; i++) {
        int nb = box_offsets[i + 1] - box_offsets[i];
        const float* bb = boxes + (size_t)box_offsets[i] * 4;
        const int32_t* bl = labels + box_offsets[i];
        float* ob = out_boxes + (size_t)i * A * 4;
        int32_t* ol = out_labels + (size_t)i * A;
        float* ious = (float*)malloc(sizeof(float) * (size_t)nb * A);
        for (int b = 0; b < nb; b++) {
            const float* box = bb + b * 4;
            float* row = ious + (size_t)b * A;
            float area = (box[3] - box[1]) * (box[2] - box[0]);
            int best = 0;
            row[0] = iou_ltrb(box, area, anchors);
            float best_iou = row[0];
            for (int a = 1; a < A; a++) {
                row[a] = iou_ltrb(box, area, anchors + a * 4);
                if (row[a] > best_iou) { best_iou = row[a]; best = a; }
            }
            row[best] = 2.f;
        }
        for (int a = 0; a < A; a++) {
            const float* an = anchors + a * 4;
            int best = 0;
            /* A sample without boxes: the reference reads the first IoU row regardless (undefined
             * behaviour there); here every anchor of such a sample is unmatched. */
            float best_iou = nb > 0 ? ious[a] : -1.f;
            for (int b = 1; b < nb; b++) {
                float v = ious[(size_t)b * A + a];
                if (v >= best_iou) { best_iou = v; best = b; }
            }
            const float* box = bb + best * 4;
            if (nb > 0 && ious[(size_t)best * A + a] > criteria) {
                float xc, yc, w, h;
                if (offset) {
                    xc = (box[0] + box[2]) * half_scale;
                    yc = (box[1] + box[3]) * half_scale;
                    w = (box[2] - box[0]) * scale;
                    h = (box[3] - box[1]) * scale;
                    float axc = (an[0] + an[2]) * half_scale, ayc = (an[1] + an[3]) * half_scale;
                    float aw = (an[2] - an[0]) * scale, ah = (an[3] - an[1]) * scale;
                    xc = ((xc - axc) / aw - means[0]) * inv_stds[0];
                    yc = ((yc - ayc) / ah - means[1]) * inv_stds[1];
                    w = (logf(w / aw) - means[2]) * inv_stds[2];
                    h = (logf(h / ah) - means[3]) * inv_stds[3];
                } else {
                    xc = (float)(0.5 * (box[0] + box[2]));
                    yc = (float)(0.5 * (box[1] + box[3]));
                    w = box[2] - box[0];
                    h = box[3] - box[1];
                }
                ob[a * 4 + 0] = xc; ob[a * 4 + 1] = yc; ob[a * 4 + 2] = w; ob[a * 4 + 3] = h;
                ol[a] = bl[best];
            } else {
                if (offset) {
                    ob[a * 4 + 0] = ob[a * 4 + 1] = ob[a * 4 + 2] = ob[a * 4 + 3] = 0.f;
                } else {
                    ob[a * 4 + 0] = (float)(0.5 * (an[0] + an[2]));
                    ob[a * 4 + 1] = (float)(0.5 * (an[1] + an[3]));
                    ob[a * 4 + 2] = -an[0] + an[2];
                    ob[a * 4 + 3] = -an[1] + an[3];
                }
                ol[a] = 0;
            }
        }
        free(ious);
    }
    return RB200_OK;
}

/* ------------------------------------------------------------------------------------------
 * Box IoU matcher. Restates BoundingBoxGraph::update_box_iou_matcher
 * (rocAL/source/meta_data/bounding_box_graph.cpp:222-284):
 *   :247-251  per anchor: the box with the highest IoU by strict '>' from -1 (lowest box index among
 *             equals; NaN never matches)
 *   :254-256  per box: the highest IoU over the anchors, by strict '>' from -1
 *   :259-264  low-quality matches: every anchor whose IoU with a box lies within 1e-6 of that box's
 *             maximum keeps its match whatever the thresholds
 *   :268-277  otherwise a best IoU below low_threshold gives -1, below high_threshold -2.
 * An anchor that no box beats (a sample without boxes, NaN IoUs) keeps the entry the reference finds in
 * its output buffer; here that entry is -1 before the threshold rules apply.
 * All pointers are host pointers.
 * ---------------------------------------------------------------------------------------- */
ORC_API int orc_box_iou_match(const float* boxes, const int32_t* box_offsets, int n, const float* anchors,
                              int num_anchors, float high_threshold, float low_threshold, int allow_low_quality,
                              int32_t* out_matches) {
    if (!boxes || !box_offsets || !anchors || !out_matches) return RB200_E_INVALID;
    int A = num_anchors;
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < n; i++) {
        int nb = box_offsets[i + 1] - box_offsets[i];
        const float* bb = boxes + (size_t)box_offsets[i] * 4;
        int32_t* m = out_matches + (size_t)i * A;
        float* vals = (float*)malloc(sizeof(float) * (size_t)A);
        float* row = (float*)malloc(sizeof(float) * (size_t)A);
        uint8_t* lq = (uint8_t*)calloc((size_t)A, 1);
        for (int a = 0; a < A; a++) { vals[a] = -1.f; m[a] = -1; }
        for (int b = 0; b < nb; b++) {
            const float* box = bb + b * 4;
            float area = (box[3] - box[1]) * (box[2] - box[0]);
            float best = -1.f;
            for (int a = 0; a < A; a++) {
                float v = iou_ltrb(box, area, anchors + a * 4);
                row[a] = v;
                if (v > vals[a]) { vals[a] = v; m[a] = b; }
                if (allow_low_quality && v > best) best = v;
            }
            if (allow_low_quality)
                for (int a = 0; a < A; a++)
                    if ((double)fabsf(row[a] - best) < 1e-6) lq[a] = 1;
        }
        for (int a = 0; a < A; a++) {
            if (!(allow_low_quality && lq[a])) {
                if (vals[a] < low_threshold) m[a] = -1;
                else if (vals[a] < high_threshold) m[a] = -2;
            }
        }
        free(vals); free(row); free(lq);
    }
    return RB200_OK;
}

/* ------------------------------------------------------------------------------------------
 * Host-side size rules.
 * ---------------------------------------------------------------------------------------- */

/* Target size of one resized sample: ResizeNode::adjust_out_roi_size
 * (rocAL/source/augmentations/geometry_augmentations/node_resize.cpp:98-138) followed by the
 * clamp to the output tensor's maximum shape (:71-72). mode follows RocalResizeScalingMode
 * (0 default, 1 stretch, 2 not-smaller, 3 not-larger, 4 min-max: ResizeMirrorNormalize only). */
ORC_API void orc_resize_dst_size(unsigned src_w, unsigned src_h, unsigned dst_w, unsigned dst_h, int mode,
                                 unsigned max_w, unsigned max_h, unsigned cap_w, unsigned cap_h,
                                 unsigned* out_w, unsigned* out_h) {
    int has_max = (max_w | max_h) > 0;
    if (mode == 4) {
        /* MIN_MAX (node_resize_mirror_normalize.cpp:138-160): max_w carries the minimum size, max_h the maximum size;
         * the shorter side becomes min_size unless the longer one would then exceed max_size; integer division. */
        unsigned min_size = max_w, max_size = max_h, size = min_size;
        float min_o = (float)(src_w < src_h ? src_w : src_h), max_o = (float)(src_w > src_h ? src_w : src_h);
        if (max_o / min_o * size > max_size) size = (unsigned)(size_t)roundf(max_size * min_o / max_o);
        if (src_w < src_h) {
            dst_w = size;
            dst_h = (unsigned)((size_t)size * src_h / src_w);
        } else {
            dst_h = size;
            dst_w = (unsigned)((size_t)size * src_w / src_h);
        }
    } else if (mode == 1) {
        if (!dst_w) dst_w = src_w;
        if (!dst_h) dst_h = src_h;
        if (has_max) {
            if (max_w) dst_w = dst_w < max_w ? dst_w : max_w;
            if (max_h) dst_h = dst_h < max_h ? dst_h : max_h;
        }
    } else if (mode == 0) {
        if ((!dst_w) & (dst_h != 0)) {
            dst_w = (unsigned)lroundf(src_w * ((float)dst_h / src_h));
        } else if ((!dst_h) & (dst_w != 0)) {
            dst_h = (unsigned)lroundf(src_h * ((float)dst_w / src_w));
        }
        if (has_max) {
            if (max_w) dst_w = dst_w < max_w ? dst_w : max_w;
            if (max_h) dst_h = dst_h < max_h ? dst_h : max_h;
        }
    } else {
        float scale = 1.0f;
        float scale_w = (float)dst_w / src_w;
        float scale_h = (float)dst_h / src_h;
        if (mode == 2) {
            scale = scale_w > scale_h ? scale_w : scale_h;
        } else if (mode == 3) {
            scale = (scale_w > 0 && scale_h > 0) ? (scale_w < scale_h ? scale_w : scale_h)
                                                 : ((scale_w > 0) ? scale_w : scale_h);
        }
        if (has_max) {
            if (max_w) scale = fminf(scale, (float)max_w / src_w);
            if (max_h) scale = fminf(scale, (float)max_h / src_h);
        }
        if ((scale_h != scale) || (!dst_h)) dst_h = (unsigned)lroundf(src_h * scale);
        if ((scale_w != scale) || (!dst_w)) dst_w = (unsigned)lroundf(src_w * scale);
    }
    *out_w = dst_w < cap_w ? dst_w : cap_w;
    *out_h = dst_h < cap_h ? dst_h : cap_h;
}

/* Fixed-anchor crop window: RocalCropParam::fill_crop_dims, non-random branch
 * (rocAL/source/parameters/parameter_rocal_crop.cpp:51-61,77-84). */
ORC_API void orc_crop_fixed(unsigned in_w, unsigned in_h, unsigned crop_w, unsigned crop_h, float anchor_x,
                            float anchor_y, unsigned* x1, unsigned* y1, unsigned* cw, unsigned* ch) {
    unsigned w = (crop_w <= in_w && crop_w > 0) ? crop_w : in_w;
    unsigned h = (crop_h <= in_h && crop_h > 0) ? crop_h : in_h;
    unsigned x = (unsigned)(size_t)nearbyintf(anchor_x * (in_w - w));
    unsigned y = (unsigned)(size_t)nearbyintf(anchor_y * (in_h - h));
    unsigned x2 = x + w, y2 = y + h;
    if (x2 > in_w) x2 = in_w;
    if (y2 > in_h) y2 = in_h;
    *x1 = x; *y1 = y; *cw = w; *ch = h;
    (void)x2; (void)y2;
}

/* ------------------------------------------------------------------------------------------
 * Normalize: out = scale * (x - mean) / stddev + shift (rocAL_pybind/amd/rocal/fn.py:1216-1223,
 * rocAL/source/augmentations/effects_augmentations/node_normalize.cpp:31-105 for the meaning of the axis mask and
 * of given / computed statistics). The reference keeps the arithmetic in RPP: PARITY UNPINNED. Definitions used
 * here: statistics of the whole population from exact integer sums, evaluated in double (mean = S1/N,
 * var = (S2 - 2 m S1)/N + m^2 about the float mean m in use, negative values from rounding count as 0), both
 * rounded to float; mult = scale / stddev in float (0 when stddev is 0); out = fmaf(x - mean, mult, shift).
 * ---------------------------------------------------------------------------------------- */
static int norm_stat_index(int mask, int y, int x, int c, int w) {
    switch (mask) {
        case 1: return x * 3 + c;
        case 2: return y * 3 + c;
        case 3: return c;
        case 4: return y * w + x;
        case 5: return x;
        case 6: return y;
        default: return 0;
    }
}

static int norm_stat_slots(int mask, int w, int h) {
    switch (mask) {
        case 1: return 3 * w;
        case 2: return 3 * h;
        case 3: return 3;
        case 4: return w * h;
        case 5: return w;
        case 6: return h;
        default: return 1;
    }
}

typedef struct orc_normalize_params {
    void* out;
    int32_t out_w, out_h, out_dtype, axis_mask, compute_mean, compute_stddev, fill_padding;
    float mean[3], stddev[3], scale, shift;
} orc_normalize_params;

ORC_API int orc_normalize(const uint8_t* arena, const rb200_pointwise_sample* s, int n, const orc_normalize_params* p) {
    if (!arena || !s || !p || !p->out || n < 0) return RB200_E_INVALID;
    const int mask = p->axis_mask & 7;
    const int computes = p->compute_mean || p->compute_stddev;
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < n; i++) {
        const rb200_pointwise_sample* q = &s[i];
        const uint8_t* img = arena + q->src_offset + (size_t)q->roi_y * q->src_stride + (size_t)q->roi_x * 3;
        const int w = q->roi_w < p->out_w ? q->roi_w : p->out_w;
        const int h = q->roi_h < p->out_h ? q->roi_h : p->out_h;
        if (p->fill_padding) {
            size_t elems = (size_t)3 * p->out_w * p->out_h, esz = p->out_dtype == RB200_FP32 ? 4 : 2;
            memset((uint8_t*)p->out + (size_t)i * elems * esz, 0, elems * esz);
        }
        if (w <= 0 || h <= 0) continue;
        const int slots = computes ? norm_stat_slots(mask, w, h) : 0;
        uint64_t* s1 = (uint64_t*)calloc((size_t)(slots > 0 ? slots : 1), sizeof(uint64_t));
        uint64_t* s2 = (uint64_t*)calloc((size_t)(slots > 0 ? slots : 1), sizeof(uint64_t));
        if (computes)
            for (int y = 0; y < h; y++)
                for (int x = 0; x < w; x++)
                    for (int c = 0; c < 3; c++) {
                        uint64_t v = img[(size_t)y * q->src_stride + x * 3 + c];
                        int k = norm_stat_index(mask, y, x, c, w);
                        s1[k] += v;
                        s2[k] += v * v;
                    }
        double cnt;
        switch (mask) {
            case 1: cnt = h; break;
            case 2: cnt = w; break;
            case 3: cnt = (double)w * h; break;
            case 4: cnt = 3.0; break;
            case 5: cnt = 3.0 * h; break;
            case 6: cnt = 3.0 * w; break;
            default: cnt = 3.0 * w * h;
        }
        for (int y = 0; y < h; y++)
            for (int x = 0; x < w; x++)
                for (int c = 0; c < 3; c++) {
                    float mean_f = p->mean[c], std_f = p->stddev[c];
                    if (computes) {
                        int k = norm_stat_index(mask, y, x, c, w);
                        int ch = (mask == 1 || mask == 2 || mask == 3) ? c : 0;
                        mean_f = p->compute_mean ? (float)((double)s1[k] / cnt) : p->mean[ch];
                        if (p->compute_stddev) {
                            double m = (double)mean_f;
                            double var = ((double)s2[k] - 2.0 * m * (double)s1[k]) / cnt + m * m;
                            if (!(var > 0.0)) var = 0.0;
                            std_f = (float)sqrt(var);
                        } else {
                            std_f = p->stddev[ch];
                        }
                    }
                    float mult = std_f > 0.f ? p->scale / std_f : 0.f;
                    float px = (float)img[(size_t)y * q->src_stride + x * 3 + c];
                    float o = fmaf(px - mean_f, mult, p->shift);
                    store_elem(p->out, p->out_dtype, (((size_t)i * p->out_h + y) * p->out_w + x) * 3 + c, o);
                }
        free(s1);
        free(s2);
    }
    return RB200_OK;
}

/* Axis permutation of the sample's h x w x 3 window: extents (d[perm[0]], d[perm[1]], d[perm[2]]) at the origin of the
 * sample's slot of out_dims[0] x out_dims[1] x out_dims[2] bytes (rocalTranspose, rocal_api_augmentation.cpp:2349-2378:
 * the output tensor's maximum shape is the permuted maximum shape of the input; pure indexing). */
ORC_API int orc_transpose(const uint8_t* arena, const rb200_pointwise_sample* s, int n, const int32_t* perm, uint8_t* out,
                          const int32_t* out_dims) {
    if (!arena || !s || !perm || !out || !out_dims) return RB200_E_INVALID;
    const int m0 = out_dims[0], m1 = out_dims[1], m2 = out_dims[2];
    for (int i = 0; i < n; i++) {
        const rb200_pointwise_sample* q = &s[i];
        const uint8_t* img = arena + q->src_offset + (size_t)q->roi_y * q->src_stride + (size_t)q->roi_x * 3;
        const int d[3] = {q->roi_h, q->roi_w, 3};
        const int o0 = d[perm[0]], o1 = d[perm[1]], o2 = d[perm[2]];
        uint8_t* o = out + (size_t)i * m0 * m1 * m2;
        for (int i0 = 0; i0 < o0 && i0 < m0; i0++)
            for (int i1 = 0; i1 < o1 && i1 < m1; i1++)
                for (int i2 = 0; i2 < o2 && i2 < m2; i2++) {
                    int idx[3];
                    idx[perm[0]] = i0; idx[perm[1]] = i1; idx[perm[2]] = i2;
                    o[((size_t)i0 * m1 + i1) * m2 + i2] = img[(size_t)idx[0] * q->src_stride + idx[1] * 3 + idx[2]];
                }
    }
    return RB200_OK;
}

ORC_API const char* orc_version(void) { return "rocal_b200 oracle 1"; }
