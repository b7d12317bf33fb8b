// Bounding boxes through a crop window and a mirror, on the device: for callers whose annotations already live in
// device memory (the pipeline itself transforms its boxes on the host, where they are born and where the window
// samplers need them, and uploads the result once).
//
// Per sample: a window {l, t, r, b} in the normalised coordinates of the boxes, a keep rule, and mirror flags.
//   rule RB200_BOX_RULE_QUARTER_AREA  the Crop / CropMirrorNormalize / ResizeCropMirror meta nodes
//        (rocAL/source/meta_data/meta_node_crop.cpp:59-78, meta_node_crop_mirror_normalize.cpp:53-90,
//        meta_node_resize_crop_mirror.cpp:66-100): a box stays when at least a quarter of its area lies in the
//        window; a sample left without boxes gets the whole window with label 0
//   rule RB200_BOX_RULE_CENTRE        the SSD / random bbox crop (bounding_box_graph.cpp:98-110): a box stays when its
//        centre lies strictly inside; a sample left without boxes gets one empty box with label 0
// Kept boxes are clipped to the window and re-normalised to it, then mirrored (meta_node_flip.cpp:40-60). Every float
// operation rounds once, in the order of the host code (pipeline.cpp: transform_boxes_window, mirror_boxes), so the
// result is bit-identical to it.
//
// Three small launches: keep counts per sample (one warp per sample), an exclusive scan of the counts into the output
// offsets (one CTA), and the compacting write (one warp per sample, order preserved by ballot prefix counts).
#include "common.cuh"

namespace rb200 {

__device__ __forceinline__ bool box_kept(const float4 q, const rb200_box_window& w, int rule) {
    if (rule == RB200_BOX_RULE_CENTRE) {
        const float xc = mul_rn(0.5f, add_rn(q.x, q.z)), yc = mul_rn(0.5f, add_rn(q.y, q.w));
        return xc > w.l && xc < w.r && yc > w.t && yc < w.b;
    }
    const float xa = fmaxf(q.x, w.l), ya = fmaxf(q.y, w.t), xb = fminf(q.z, w.r), yb = fminf(q.w, w.b);
    const float inter = mul_rn(fmaxf(0.f, sub_rn(xb, xa)), fmaxf(0.f, sub_rn(yb, ya)));
    const float area = mul_rn(sub_rn(q.w, q.y), sub_rn(q.z, q.x));
    return div_rn(inter, area) >= 0.25f;        // 0 / 0 (an empty box) is NaN and drops the box, as on the host
}

constexpr int kBoxWarps = 8;    // samples per CTA

__global__ void __launch_bounds__(kBoxWarps * 32) box_keep_count_kernel(const float4* __restrict__ boxes,
                                                                        const int* __restrict__ offsets, int n,
                                                                        const rb200_box_window* __restrict__ windows, int rule,
                                                                        int* __restrict__ out_offsets) {
    const int i = blockIdx.x * kBoxWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= n) return;
    const int b0 = offsets[i], nb = offsets[i + 1] - b0;
    const rb200_box_window w = windows[i];
    int kept = 0;
    for (int j0 = 0; j0 < nb; j0 += 32) {
        const int j = j0 + lane;
        const bool k = j < nb && box_kept(boxes[b0 + j], w, rule);
        kept += __popc(__ballot_sync(0xffffffffu, k));
    }
    if (lane == 0) out_offsets[i + 1] = kept > 0 ? kept : 1;     // a sample without boxes gets a stand-in
    if (i == 0 && lane == 0) out_offsets[0] = 0;
}

// In-place inclusive scan of out_offsets[1..n] by one CTA: every thread sums a contiguous chunk, the chunk totals are
// scanned in shared memory, the chunks are rewritten with their running sums.
__global__ void __launch_bounds__(1024) box_offsets_scan_kernel(int* __restrict__ out_offsets, int n) {
    __shared__ int totals[1024];
    const int t = threadIdx.x;
    const int chunk = (n + 1023) / 1024;
    const int lo = 1 + t * chunk, hi = min(lo + chunk, n + 1);
    int sum = 0;
    for (int i = lo; i < hi; i++) sum += out_offsets[i];
    totals[t] = sum;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {
        const int v = t >= d ? totals[t - d] : 0;
        __syncthreads();
        totals[t] += v;
        __syncthreads();
    }
    int run = totals[t] - sum;
    for (int i = lo; i < hi; i++) {
        run += out_offsets[i];
        out_offsets[i] = run;
    }
}

__global__ void __launch_bounds__(kBoxWarps * 32) box_write_kernel(const float4* __restrict__ boxes, const int* __restrict__ labels,
                                                                   const int* __restrict__ offsets, int n,
                                                                   const rb200_box_window* __restrict__ windows, int rule,
                                                                   const int* __restrict__ out_offsets, float4* __restrict__ out_boxes,
                                                                   int* __restrict__ out_labels) {
    const int i = blockIdx.x * kBoxWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= n) return;
    const int b0 = offsets[i], nb = offsets[i + 1] - b0;
    const rb200_box_window w = windows[i];
    const float ww = sub_rn(w.r, w.l), wh = sub_rn(w.b, w.t);
    const int o0 = out_offsets[i];
    int kept = 0;
    for (int j0 = 0; j0 < nb; j0 += 32) {
        const int j = j0 + lane;
        float4 q = j < nb ? boxes[b0 + j] : make_float4(0.f, 0.f, 0.f, 0.f);
        const bool k = j < nb && box_kept(q, w, rule);
        const unsigned m = __ballot_sync(0xffffffffu, k);
        if (k) {
            float4 r;
            r.x = div_rn(sub_rn(fmaxf(q.x, w.l), w.l), ww);
            r.y = div_rn(sub_rn(fmaxf(q.y, w.t), w.t), wh);
            r.z = div_rn(sub_rn(fminf(q.z, w.r), w.l), ww);
            r.w = div_rn(sub_rn(fminf(q.w, w.b), w.t), wh);
            if (w.mirror_h) { const float l = sub_rn(1.0f, r.z), rr = sub_rn(1.0f, r.x); r.x = l; r.z = rr; }
            if (w.mirror_v) { const float t = sub_rn(1.0f, r.w), bb = sub_rn(1.0f, r.y); r.y = t; r.w = bb; }
            const int pos = o0 + kept + __popc(m & ((1u << lane) - 1u));
            out_boxes[pos] = r;
            out_labels[pos] = labels[b0 + j];
        }
        kept += __popc(m);
    }
    if (kept == 0 && lane == 0) {
        float4 r = rule == RB200_BOX_RULE_CENTRE ? make_float4(0.f, 0.f, 0.f, 0.f) : make_float4(0.f, 0.f, 1.f, 1.f);
        if (w.mirror_h) { const float l = sub_rn(1.0f, r.z), rr = sub_rn(1.0f, r.x); r.x = l; r.z = rr; }
        if (w.mirror_v) { const float t = sub_rn(1.0f, r.w), bb = sub_rn(1.0f, r.y); r.y = t; r.w = bb; }
        out_boxes[o0] = r;
        out_labels[o0] = 0;
    }
}

}  // namespace rb200

using namespace rb200;

extern "C" int rb200k_box_transform(const float* boxes, const int32_t* labels, const int32_t* box_offsets, int n,
                                    const rb200_box_window* windows, int rule, float* out_boxes, int32_t* out_labels,
                                    int32_t* out_offsets, void* stream_v) {
    if (n == 0) return RB200_OK;
    if (!box_offsets || !windows || !out_boxes || !out_labels || !out_offsets || n < 0) {
        set_error("rb200k_box_transform: null pointer or negative size");
        return RB200_E_INVALID;
    }
    if (rule != RB200_BOX_RULE_QUARTER_AREA && rule != RB200_BOX_RULE_CENTRE) {
        set_error("rb200k_box_transform: bad rule %d", rule);
        return RB200_E_INVALID;
    }
    if (n > 65535) {
        set_error("rb200k_box_transform: batch %d exceeds 65535", n);
        return RB200_E_LIMIT;
    }
    if (((uintptr_t)boxes | (uintptr_t)out_boxes) & 15) {
        set_error("rb200k_box_transform: boxes and out_boxes must be 16-byte aligned");
        return RB200_E_INVALID;
    }
    cudaStream_t stream = (cudaStream_t)stream_v;
    const float4* b4 = reinterpret_cast<const float4*>(boxes);
    const unsigned ctas = (unsigned)((n + kBoxWarps - 1) / kBoxWarps);
    box_keep_count_kernel<<<ctas, kBoxWarps * 32, 0, stream>>>(b4, box_offsets, n, windows, rule, out_offsets);
    RB200_CHECK_LAUNCH("box_keep_count_kernel");
    box_offsets_scan_kernel<<<1, 1024, 0, stream>>>(out_offsets, n);
    RB200_CHECK_LAUNCH("box_offsets_scan_kernel");
    box_write_kernel<<<ctas, kBoxWarps * 32, 0, stream>>>(b4, labels, box_offsets, n, windows, rule, out_offsets,
                                                          reinterpret_cast<float4*>(out_boxes), out_labels);
    RB200_CHECK_LAUNCH("box_write_kernel");
    return RB200_OK;
}
