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

}  // extern "C"

// Stand-ins for the OpenVX array calls that the crop parameter classes make when they mirror their vectors into
// vx_arrays (never reached by the entry points above, which read the vectors).
extern "C" {
vx_context vxGetContext(vx_reference) { return nullptr; }
vx_array vxCreateArray(vx_context, vx_enum, vx_size) { return nullptr; }
vx_status vxAddArrayItems(vx_array, vx_size, const void*, vx_size) { return 0; }
vx_status vxCopyArrayRange(vx_array, vx_size, vx_size, vx_size, void*, vx_enum, vx_enum) { return 0; }
}
