/*
 * ref_driver.cpp — C entry points around reference-owned CPU code. TEST INFRASTRUCTURE ONLY.
 *
 * Built by oracle/build.py together with the reference's own
 * rocAL/source/meta_data/bounding_box_graph.cpp, compiled where it lies in the reference
 * tree (nothing of the reference is copied here). The result, oracle/_ref/libref.so, is used
 * to pin the restatement in oracle.c, to generate the golden vectors under tests/golden/ and
 * as the "reference" CPU baseline of the box encoder.
 *
 *   ref_box_encode       -> BoundingBoxGraph::update_box_encoder_meta_data
 *                           (rocAL/source/meta_data/bounding_box_graph.cpp:150-220)
 *   ref_box_iou_match    -> BoundingBoxGraph::update_box_iou_matcher (bounding_box_graph.cpp:222-284);
 *                           the output buffer is pre-filled with -1 (the reference leaves unmatched entries as found)
 *   ref_uniform_rand_*   -> UniformRand<T> (rocAL/include/parameters/parameter_random.h:37-116)
 *   ref_custom_rand_int  -> CustomRand<int> (parameter_random.h:118-239)
 *   ref_seed_sequence    -> the seed table of ParameterFactory::set_seed
 *                           (rocAL/source/parameters/parameter_factory.cpp:114-119)
 *   ref_random_crop_windows -> RocalRandomCropDecParam::generate_random_seeds + generate_crop_window
 *                           (rocAL/source/parameters/parameter_random_crop_decoder.cpp:41-108, compiled in place
 *                           with parameter_factory.cpp); the batch seed is the reference's own std::random_device
 *                           draw and is handed back so that a restatement can start from the same value
 *   ref_random_area_windows -> RocalRandomCropParam::fill_crop_dims (rocAL/source/parameters/parameter_random_crop.cpp:48-97,
 *                           compiled in place with parameter_crop.cpp) with fixed or default-range parameters; the OpenVX
 *                           array calls of the class are answered by the do-nothing stand-ins at the end of this file
 *   ref_rocal_crop_windows  -> RocalCropParam::update_array -> fill_crop_dims (rocAL/source/parameters/
 *                           parameter_rocal_crop.cpp:45-85): the window rule of rocalCrop / rocalCropFixed /
 *                           rocalCropCenterFixed / rocalCropMirrorNormalize / rocalResizeCropMirror
 *   ref_random_bbox_meta    -> BoundingBoxGraph::update_random_bbox_meta_data (bounding_box_graph.cpp:71-118): boxes
 *                           that follow a crop window (centre-inside mask, clip, shift)
 */
#include <cstdint>
#include <memory>
#include <random>
#include <vector>

#include "meta_data/bounding_box_graph.h"
#include "parameters/parameter_factory.h"
#include "parameters/parameter_random.h"
#include "parameters/parameter_random_crop.h"
#include "parameters/parameter_random_crop_decoder.h"
#include "parameters/parameter_rocal_crop.h"

extern "C" {

__attribute__((visibility("default"))) int ref_box_encode(
    const float* boxes, const int32_t* labels, const int32_t* box_offsets, int n, const float* anchors,
    int num_anchors, float criteria, const float* means, const float* stds, int offset, float scale,
    float* out_boxes, int32_t* out_labels) {
    auto batch = std::make_shared<BoundingBoxBatch>();
    batch->resize(n);
    for (int i = 0; i < n; i++) {
        BoundingBoxCords cords;
        Labels lab;
        for (int b = box_offsets[i]; b < box_offsets[i + 1]; b++) {
            cords.emplace_back(boxes[b * 4 + 0], boxes[b * 4 + 1], boxes[b * 4 + 2], boxes[b * 4 + 3]);
            lab.push_back(labels[b]);
        }
        batch->get_bb_cords_batch()[i] = cords;
        batch->get_labels_batch()[i] = lab;
    }
    std::vector<float> anc(anchors, anchors + (size_t)num_anchors * 4);
    std::vector<float> m(means, means + 4), s(stds, stds + 4);
    BoundingBoxGraph graph;
    graph.update_box_encoder_meta_data(&anc, batch, criteria, offset != 0, scale, m, s, out_boxes, out_labels);
    return 0;
}

__attribute__((visibility("default"))) int ref_box_iou_match(
    const float* boxes, const int32_t* box_offsets, int n, const float* anchors, int num_anchors,
    float high_threshold, float low_threshold, int allow_low_quality, int32_t* out_matches) {
    auto batch = std::make_shared<BoundingBoxBatch>();
    batch->resize(n);
    for (int i = 0; i < n; i++) {
        BoundingBoxCords cords;
        Labels lab;
        for (int b = box_offsets[i]; b < box_offsets[i + 1]; b++) {
            cords.emplace_back(boxes[b * 4 + 0], boxes[b * 4 + 1], boxes[b * 4 + 2], boxes[b * 4 + 3]);
            lab.push_back(0);
        }
        batch->get_bb_cords_batch()[i] = cords;
        batch->get_labels_batch()[i] = lab;
    }
    std::vector<float> anc(anchors, anchors + (size_t)num_anchors * 4);
    BoxIouMatcherInfo info;
    info.anchors = &anc;
    info.high_threshold = high_threshold;
    info.low_threshold = low_threshold;
    info.allow_low_quality_matches = allow_low_quality != 0;
    for (size_t k = 0; k < (size_t)n * num_anchors; k++) out_matches[k] = -1;
    BoundingBoxGraph graph;
    graph.update_box_iou_matcher(info, out_matches, batch);
    return 0;
}

/* `batches` renewals of a length-`batch` array, as MasterGraph::update_node_parameters does once
 * per batch (rocAL/source/pipeline/master_graph.cpp:405-415); out holds batches*batch values. */
__attribute__((visibility("default"))) void ref_uniform_rand_float(unsigned seed, float start, float end,
                                                                    unsigned batch, unsigned batches, float* out) {
    UniformRand<float> p(start, end, seed);
    p.create_array(batch);
    for (unsigned b = 0; b < batches; b++) {
        p.renew();
        auto v = p.get_array();
        for (unsigned i = 0; i < batch; i++) out[b * batch + i] = v[i];
    }
}

__attribute__((visibility("default"))) void ref_uniform_rand_int(unsigned seed, int start, int end, unsigned batch,
                                                                  unsigned batches, int* out) {
    UniformRand<int> p(start, end, seed);
    p.create_array(batch);
    for (unsigned b = 0; b < batches; b++) {
        p.renew();
        auto v = p.get_array();
        for (unsigned i = 0; i < batch; i++) out[b * batch + i] = v[i];
    }
}

__attribute__((visibility("default"))) void ref_custom_rand_int(unsigned seed, const int* values,
                                                                 const double* freqs, unsigned size, unsigned batch,
                                                                 unsigned batches, int* out) {
    CustomRand<int> p(values, freqs, size, seed);
    p.create_array(batch);
    for (unsigned b = 0; b < batches; b++) {
        p.renew();
        auto v = p.get_array();
        for (unsigned i = 0; i < batch; i++) out[b * batch + i] = v[i];
    }
}

__attribute__((visibility("default"))) void ref_seed_sequence(unsigned seed, unsigned count, int64_t* out) {
    std::vector<int64_t> table(count);
    std::seed_seq ss{seed};
    ss.generate(table.begin(), table.end());
    for (unsigned i = 0; i < count; i++) out[i] = table[i];
}

// shapes_hw: n x {height, width}; out_xywh: n x {x, y, w, h}; returns the batch seed the windows came from.
__attribute__((visibility("default"))) unsigned ref_random_crop_windows(const int* shapes_hw, int n, float aspect_lo,
                                                                        float aspect_hi, float area_lo, float area_hi,
                                                                        int num_attempts, unsigned* out_xywh) {
    RocalRandomCropDecParam param({aspect_lo, aspect_hi}, {area_lo, area_hi}, 0, num_attempts, n);
    param.generate_random_seeds();
    const unsigned batch_seed = ParameterFactory::instance()->get_seed();
    for (int i = 0; i < n; i++) {
        Shape shape = {(size_t)shapes_hw[i * 2], (size_t)shapes_hw[i * 2 + 1]};
        CropWindow w = param.generate_crop_window(shape, i);
        out_xywh[i * 4 + 0] = w.x;
        out_xywh[i * 4 + 1] = w.y;
        out_xywh[i * 4 + 2] = w.W;
        out_xywh[i * 4 + 3] = w.H;
    }
    return batch_seed;
}

// wh: n x {width, height}; out_xywh: n x {x, y, w, h}. fixed != 0: the four values of `fixed4` = {area, aspect,
// x_drift, y_drift} as single-value parameters; fixed == 0: ParameterFactory::set_seed(seed) and the class's own
// default uniform ranges. Every construction of the class takes the next four entries of the seed table for x_drift,
// y_drift, area and aspect in that order (set_seed does not rewind the table), so the index of the first entry this
// call used is returned.
namespace {
struct RandomAreaProbe : public RocalRandomCropParam {
    using RocalRandomCropParam::RocalRandomCropParam;
    using RocalRandomCropParam::set_area_factor;
    using RocalRandomCropParam::set_aspect_ratio;
    using RocalRandomCropParam::fill_crop_dims;
};
}  // namespace

__attribute__((visibility("default"))) unsigned ref_random_area_windows(const unsigned* wh, int n, int fixed, const float* fixed4,
                                                                        unsigned seed, unsigned* out_xywh) {
    static unsigned constructions = 0;
    const unsigned first_entry = (constructions++ * 4u) % 1024u;
    ParameterFactory* f = ParameterFactory::instance();
    if (!fixed) f->set_seed(seed);
    RandomAreaProbe p((unsigned)n);
    if (fixed) {
        p.set_area_factor(f->create_single_value_param(fixed4[0]));
        p.set_aspect_ratio(f->create_single_value_param(fixed4[1]));
        p.set_x_drift_factor(f->create_single_value_param(fixed4[2]));
        p.set_y_drift_factor(f->create_single_value_param(fixed4[3]));
    }
    std::vector<Roi2DCords> rois(n);
    for (int i = 0; i < n; i++) {
        rois[i].xywh.x = 0;
        rois[i].xywh.y = 0;
        rois[i].xywh.w = wh[i * 2];
        rois[i].xywh.h = wh[i * 2 + 1];
    }
    p.array_init();
    p.set_image_dimensions(rois.data());
    p.fill_crop_dims();
    auto x1 = p.get_x1_arr_val(), y1 = p.get_y1_arr_val(), cw = p.get_cropw_arr_val(), ch = p.get_croph_arr_val();
    for (int i = 0; i < n; i++) {
        out_xywh[i * 4 + 0] = x1[i];
        out_xywh[i * 4 + 1] = y1[i];
        out_xywh[i * 4 + 2] = cw[i];
        out_xywh[i * 4 + 3] = ch[i];
    }
    return first_entry;
}

// wh: n x {width, height} of the input ROIs. mode 0: fixed anchors (set_fixed_crop(f[0], f[1]), crop size crop_w x crop_h);
// mode 1: absolute corner x1 = f[0], y1 = f[1] (neither fixed nor random); mode 2: random branch with the single-value
// factors f = {width factor, height factor, x drift, y drift}. out: n x {x1, y1, crop_w, crop_h, x2, y2}.
namespace {
struct RocalCropProbe : public RocalCropParam {
    using RocalCropParam::RocalCropParam;
    std::vector<uint32_t> x2v() { return x2_arr_val; }
    std::vector<uint32_t> y2v() { return y2_arr_val; }
};
}  // namespace

__attribute__((visibility("default"))) int ref_rocal_crop_windows(const unsigned* wh, int n, int mode, unsigned crop_w,
                                                                  unsigned crop_h, const float* f, unsigned* out) {
    ParameterFactory* pf = ParameterFactory::instance();
    pf->set_seed(1);   // the class's default parameters take entries of the seed table, which must exist
    RocalCropProbe p((unsigned)n);
    p.crop_w = crop_w;
    p.crop_h = crop_h;
    p.x1 = p.y1 = 0;
    if (mode == 0) {
        p.set_fixed_crop(f[0], f[1]);
    } else if (mode == 1) {
        p.x1 = (unsigned)f[0];
        p.y1 = (unsigned)f[1];
    } else {
        p.set_random();
        p.set_crop_width_factor(pf->create_single_value_param(f[0]));
        p.set_crop_height_factor(pf->create_single_value_param(f[1]));
        p.set_x_drift_factor(pf->create_single_value_param(f[2]));
        p.set_y_drift_factor(pf->create_single_value_param(f[3]));
    }
    std::vector<Roi2DCords> rois(n);
    for (int i = 0; i < n; i++) {
        rois[i].xywh.x = 0;
        rois[i].xywh.y = 0;
        rois[i].xywh.w = wh[i * 2];
        rois[i].xywh.h = wh[i * 2 + 1];
    }
    p.array_init();
    p.set_image_dimensions(rois.data());
    p.update_array();
    auto x1 = p.get_x1_arr_val(), y1 = p.get_y1_arr_val(), cw = p.get_cropw_arr_val(), ch = p.get_croph_arr_val();
    auto x2 = p.x2v(), y2 = p.y2v();
    for (int i = 0; i < n; i++) {
        out[i * 6 + 0] = x1[i];
        out[i * 6 + 1] = y1[i];
        out[i * 6 + 2] = cw[i];
        out[i * 6 + 3] = ch[i];
        out[i * 6 + 4] = x2[i];
        out[i * 6 + 5] = y2[i];
    }
    return 0;
}

// boxes: [total][4] ltrb, labels [total], box_offsets [n+1]; crop_xywh: n x {x, y, w, h} as the random-bbox-crop reader
// reports them; roi_wh: n x {roi width, roi height} of the decoded images. out_boxes / out_labels hold at most
// max(total, n) entries; out_counts[n]. Returns the number of boxes written.
__attribute__((visibility("default"))) int ref_random_bbox_meta(const float* boxes, const int32_t* labels,
                                                                const int32_t* box_offsets, int n, const float* crop_xywh,
                                                                const uint32_t* roi_wh, float* out_boxes,
                                                                int32_t* out_labels, int32_t* out_counts) {
    auto in = std::make_shared<BoundingBoxBatch>();
    auto out = std::make_shared<BoundingBoxBatch>();
    in->resize(n);
    out->resize(n);
    DecodedDataInfo info;
    CropImageInfo crops;
    for (int i = 0; i < n; i++) {
        BoundingBoxCords cords;
        Labels lab;
        for (int b = box_offsets[i]; b < box_offsets[i + 1]; b++) {
            cords.emplace_back(boxes[b * 4 + 0], boxes[b * 4 + 1], boxes[b * 4 + 2], boxes[b * 4 + 3]);
            lab.push_back(labels[b]);
        }
        in->get_bb_cords_batch()[i] = cords;
        in->get_labels_batch()[i] = lab;
        info._roi_width.push_back(roi_wh[i * 2]);
        info._roi_height.push_back(roi_wh[i * 2 + 1]);
        info._original_width.push_back(roi_wh[i * 2]);
        info._original_height.push_back(roi_wh[i * 2 + 1]);
        crops._crop_image_coords.push_back({crop_xywh[i * 4], crop_xywh[i * 4 + 1], crop_xywh[i * 4 + 2], crop_xywh[i * 4 + 3]});
    }
    BoundingBoxGraph graph;
    graph.update_random_bbox_meta_data(in, out, info, crops);
    int k = 0;
    for (int i = 0; i < n; i++) {
        auto& c = out->get_bb_cords_batch()[i];
        auto& l = out->get_labels_batch()[i];
        out_counts[i] = (int)c.size();
        for (size_t j = 0; j < c.size(); j++, k++) {
            out_boxes[k * 4 + 0] = c[j].l;
            out_boxes[k * 4 + 1] = c[j].t;
            out_boxes[k * 4 + 2] = c[j].r;
            out_boxes[k * 4 + 3] = c[j].b;
            out_labels[k] = l[j];
        }
    }
    return k;
}

}  // extern "C"

// Stand-ins for the OpenVX array calls that the crop parameter classes make when they mirror their vectors into
// vx_arrays (never reached by the entry points above, which read the vectors).
extern "C" {
vx_context vxGetContext(vx_reference) { return nullptr; }
vx_array vxCreateArray(vx_context, vx_enum, vx_size) { return nullptr; }
vx_status vxAddArrayItems(vx_array, vx_size, const void*, vx_size) { return 0; }
vx_status vxCopyArrayRange(vx_array, vx_size, vx_size, vx_size, void*, vx_enum, vx_enum) { return 0; }
}
