// rocAL-signature entry points (include/rocal_api.h): thin shims that flatten std::vector arguments
// and forward to the plain C ABI in rb200_api.cpp, which owns validation and error capture.
#include <iostream>

#include "pipeline.h"

using namespace rb200;

namespace {
inline unsigned vec_at(const std::vector<unsigned>& v, size_t i) { return v.size() == 1 ? v[0] : (i < v.size() ? v[i] : 0); }
inline Pipeline* P(RocalContext c) { return static_cast<Pipeline*>(c); }
}  // namespace

extern "C" {

RocalContext ROCAL_API_CALL rocalCreate(size_t batch_size, RocalProcessMode affinity, int gpu_id, size_t cpu_thread_count,
                                        size_t prefetch_queue_depth, RocalTensorOutputType output_tensor_data_type) {
    return rb200_create(batch_size, (int)affinity, gpu_id, cpu_thread_count, prefetch_queue_depth, (int)output_tensor_data_type);
}
RocalStatus ROCAL_API_CALL rocalVerify(RocalContext context) { return (RocalStatus)rb200_verify(context); }
RocalStatus ROCAL_API_CALL rocalRun(RocalContext context) { return (RocalStatus)rb200_run(context); }
RocalStatus ROCAL_API_CALL rocalRelease(RocalContext context) { return (RocalStatus)rb200_release(context); }

void ROCAL_API_CALL rocalSetSeed(unsigned seed) { rb200_set_seed(seed); }
unsigned ROCAL_API_CALL rocalGetSeed() { return rb200_get_seed(); }
RocalIntParam ROCAL_API_CALL rocalCreateIntUniformRand(int start, int end) { return rb200_create_int_uniform_rand(start, end); }
RocalStatus ROCAL_API_CALL rocalUpdateIntUniformRand(int start, int end, RocalIntParam p) { return (RocalStatus)rb200_update_int_uniform_rand(start, end, p); }
int ROCAL_API_CALL rocalGetIntValue(RocalIntParam p) { return rb200_get_int_value(p); }
float ROCAL_API_CALL rocalGetFloatValue(RocalFloatParam p) { return rb200_get_float_value(p); }
RocalFloatParam ROCAL_API_CALL rocalCreateFloatUniformRand(float start, float end) { return rb200_create_float_uniform_rand(start, end); }
RocalFloatParam ROCAL_API_CALL rocalCreateFloatParameter(float val) { return rb200_create_float_parameter(val); }
RocalIntParam ROCAL_API_CALL rocalCreateIntParameter(int val) { return rb200_create_int_parameter(val); }
RocalStatus ROCAL_API_CALL rocalUpdateFloatParameter(float v, RocalFloatParam p) { return (RocalStatus)rb200_update_float_parameter(v, p); }
RocalStatus ROCAL_API_CALL rocalUpdateIntParameter(int v, RocalIntParam p) { return (RocalStatus)rb200_update_int_parameter(v, p); }
RocalStatus ROCAL_API_CALL rocalUpdateFloatUniformRand(float s, float e, RocalFloatParam p) { return (RocalStatus)rb200_update_float_uniform_rand(s, e, p); }
RocalIntParam ROCAL_API_CALL rocalCreateIntRand(const int* values, const double* frequencies, unsigned size) { return rb200_create_int_rand(values, frequencies, size); }
RocalFloatParam ROCAL_API_CALL rocalCreateFloatRand(const float* values, const double* frequencies, unsigned size) { return rb200_create_float_rand(values, frequencies, size); }
RocalStatus ROCAL_API_CALL rocalUpdateIntRand(const int* values, const double* frequencies, unsigned size, RocalIntParam p) {
    if (!p || !ParameterFactory::instance().owns(p)) return ROCAL_UPDATE_PARAMETER_FAILED;
    auto* h = static_cast<IntParam*>(p);
    if (h->kind != ParamKind::RANDOM_CUSTOM) return ROCAL_INVALID_PARAMETER_TYPE;
    return static_cast<CustomRand<int>*>(h->core)->update(values, frequencies, size) == 0 ? ROCAL_OK : ROCAL_UPDATE_PARAMETER_FAILED;
}
RocalStatus ROCAL_API_CALL rocalUpdateFloatRand(const float* values, const double* frequencies, unsigned size, RocalFloatParam p) {
    if (!p || !ParameterFactory::instance().owns(p)) return ROCAL_UPDATE_PARAMETER_FAILED;
    auto* h = static_cast<FloatParam*>(p);
    if (h->kind != ParamKind::RANDOM_CUSTOM) return ROCAL_INVALID_PARAMETER_TYPE;
    return static_cast<CustomRand<float>*>(h->core)->update(values, frequencies, size) == 0 ? ROCAL_OK : ROCAL_UPDATE_PARAMETER_FAILED;
}

RocalTensor ROCAL_API_CALL rocalJpegExternalFileSource(RocalContext ctx, RocalImageColor color, bool is_output, bool, bool,
                                                       RocalImageSizeEvaluationPolicy, unsigned max_width, unsigned max_height,
                                                       RocalDecoderType, RocalExternalSourceMode mode, RocalShardingInfo) {
    return static_cast<RocalTensor>(rb200_external_source(ctx, (int)color, is_output, max_width, max_height, (int)mode));
}

RocalTensor ROCAL_API_CALL rocalJpegFileSourceSingleShard(RocalContext ctx, const char* source_path, RocalImageColor color,
                                                          unsigned shard_id, unsigned shard_count, bool is_output, bool shuffle,
                                                          bool loop, RocalImageSizeEvaluationPolicy, unsigned max_width,
                                                          unsigned max_height, RocalDecoderType, RocalShardingInfo si) {
    return static_cast<RocalTensor>(rb200_jpeg_file_source(ctx, source_path, (int)color, shard_id, shard_count, is_output, shuffle, loop,
                                                           max_width, max_height, (int)si.last_batch_policy, si.pad_last_batch_repeated));
}
RocalTensor ROCAL_API_CALL rocalJpegFileSource(RocalContext ctx, const char* source_path, RocalImageColor color,
                                               unsigned internal_shard_count, bool is_output, bool shuffle, bool loop,
                                               RocalImageSizeEvaluationPolicy p, unsigned max_width, unsigned max_height,
                                               RocalDecoderType d, RocalShardingInfo si) {
    if (internal_shard_count != 1) {
        if (ctx) P(ctx)->capture_error("rocalJpegFileSource: internal_shard_count must be 1 (one context drives one GPU; use rocalJpegFileSourceSingleShard per rank)");
        return nullptr;
    }
    return rocalJpegFileSourceSingleShard(ctx, source_path, color, 0, 1, is_output, shuffle, loop, p, max_width, max_height, d, si);
}
RocalTensor ROCAL_API_CALL rocalFusedJpegCropSingleShard(RocalContext ctx, const char* source_path, RocalImageColor color,
                                                         unsigned shard_id, unsigned shard_count, bool is_output,
                                                         std::vector<float>& area_factor, std::vector<float>& aspect_ratio,
                                                         unsigned num_attempts, bool shuffle, bool loop,
                                                         RocalImageSizeEvaluationPolicy, unsigned max_width, unsigned max_height,
                                                         RocalShardingInfo si) {
    if (area_factor.size() != 2 || aspect_ratio.size() != 2) {
        if (ctx) P(ctx)->capture_error("rocalFusedJpegCrop: area_factor and aspect_ratio must hold two values each");
        return nullptr;
    }
    return static_cast<RocalTensor>(rb200_fused_jpeg_crop_file_source(ctx, source_path, (int)color, shard_id, shard_count, is_output,
                                                                      area_factor.data(), aspect_ratio.data(), num_attempts, shuffle,
                                                                      loop, max_width, max_height, (int)si.last_batch_policy,
                                                                      si.pad_last_batch_repeated));
}
RocalTensor ROCAL_API_CALL rocalFusedJpegCrop(RocalContext ctx, const char* source_path, RocalImageColor color, unsigned num_threads,
                                              bool is_output, std::vector<float>& area_factor, std::vector<float>& aspect_ratio,
                                              unsigned num_attempts, bool shuffle, bool loop, RocalImageSizeEvaluationPolicy p,
                                              unsigned max_width, unsigned max_height, RocalShardingInfo si) {
    if (num_threads != 1) {
        if (ctx) P(ctx)->capture_error("rocalFusedJpegCrop: num_threads (internal shards) must be 1 (one context drives one GPU; use rocalFusedJpegCropSingleShard per rank)");
        return nullptr;
    }
    return rocalFusedJpegCropSingleShard(ctx, source_path, color, 0, 1, is_output, area_factor, aspect_ratio, num_attempts, shuffle,
                                         loop, p, max_width, max_height, si);
}
// The folder reader numbers the classes itself; the label reader call only has to name the same folder
// (the reference keys labels by file name, label_reader_folders.cpp:95-137).
RocalMetaData ROCAL_API_CALL rocalCreateLabelReader(RocalContext ctx, const char* source_path, const char* file_list_path) {
    if (!ctx) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return nullptr;
    }
    // with a file list the following source reads the listed files in the list's order with the list's labels
    if (file_list_path && file_list_path[0]) rb200_set_file_list(ctx, file_list_path);
    (void)source_path;
    return nullptr;
}
RocalMetaData ROCAL_API_CALL rocalCreateTextFileBasedLabelReader(RocalContext ctx, const char* source_path) {
    if (!ctx) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return nullptr;
    }
    if (!source_path || !source_path[0]) {
        P(ctx)->capture_error("rocalCreateTextFileBasedLabelReader: empty path");
        return nullptr;
    }
    rb200_set_file_list(ctx, source_path);
    return nullptr;
}
// rocalCreateCOCOReader records the annotation file; the source call that follows builds the reader. Masks,
// aspect-ratio grouping and xywh output are not supported.
RocalMetaData ROCAL_API_CALL rocalCreateCOCOReader(RocalContext ctx, const char* source_path, bool is_output, bool mask, bool ltrb,
                                                   bool is_box_encoder, bool avoid_class_remapping, bool aspect_ratio_grouping,
                                                   bool is_box_iou_matcher) {
    (void)is_output; (void)is_box_encoder; (void)is_box_iou_matcher;
    if (!ctx) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return nullptr;
    }
    if (!source_path || mask || !ltrb || aspect_ratio_grouping) {
        P(ctx)->capture_error("rocalCreateCOCOReader: needs an annotation path; masks, xywh boxes and aspect-ratio grouping are not supported");
        return nullptr;
    }
    P(ctx)->note_coco_reader(source_path, avoid_class_remapping);
    return nullptr;
}
RocalTensor ROCAL_API_CALL rocalJpegCOCOFileSourceSingleShard(RocalContext ctx, const char* source_path, const char* json_path,
                                                              RocalImageColor color, unsigned shard_id, unsigned shard_count,
                                                              bool is_output, bool shuffle, bool loop, RocalImageSizeEvaluationPolicy,
                                                              unsigned max_width, unsigned max_height, RocalDecoderType, RocalShardingInfo si) {
    if (!ctx) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return nullptr;
    }
    const std::string json = (json_path && json_path[0]) ? std::string(json_path) : P(ctx)->coco_json();
    return static_cast<RocalTensor>(rb200_coco_file_source(ctx, source_path, json.c_str(), (int)color, shard_id, shard_count, is_output, shuffle,
                                                           loop, max_width, max_height, (int)si.last_batch_policy,
                                                           si.pad_last_batch_repeated, P(ctx)->coco_avoid_remap()));
}
RocalTensor ROCAL_API_CALL rocalJpegCOCOFileSource(RocalContext ctx, const char* source_path, const char* json_path, RocalImageColor color,
                                                   unsigned internal_shard_count, bool is_output, bool shuffle, bool loop,
                                                   RocalImageSizeEvaluationPolicy p, unsigned max_width, unsigned max_height,
                                                   RocalDecoderType d, RocalShardingInfo si) {
    if (internal_shard_count != 1) {
        if (ctx) P(ctx)->capture_error("rocalJpegCOCOFileSource: internal_shard_count must be 1 (use the SingleShard call per rank)");
        return nullptr;
    }
    return rocalJpegCOCOFileSourceSingleShard(ctx, source_path, json_path, color, 0, 1, is_output, shuffle, loop, p, max_width, max_height, d, si);
}
// The COCO source behind the random-crop decoder (rocal_api_data_loaders.cpp:1185-1240: the COCO storage feeds the
// fused-crop loader node). The decode window cuts the pixels only; the boxes stay those of the whole image, as in
// the reference, where only rocalRandomBBoxCrop moves boxes with a decode window (image_read_and_decode.cpp:276-329).
RocalTensor ROCAL_API_CALL rocalJpegCOCOFileSourcePartialSingleShard(RocalContext ctx, const char* source_path, const char* json_path,
                                                                     RocalImageColor color, unsigned shard_id, unsigned shard_count,
                                                                     bool is_output, std::vector<float>& area_factor,
                                                                     std::vector<float>& aspect_ratio, unsigned num_attempts, bool shuffle,
                                                                     bool loop, RocalImageSizeEvaluationPolicy p, unsigned max_width,
                                                                     unsigned max_height, RocalShardingInfo si) {
    if (!ctx) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return nullptr;
    }
    if (area_factor.size() != 2 || aspect_ratio.size() != 2) {
        P(ctx)->capture_error("rocalJpegCOCOFileSourcePartial: area_factor and aspect_ratio must hold two values each");
        return nullptr;
    }
    if (is_output) {
        P(ctx)->capture_error("rocalJpegCOCOFileSourcePartial: the fused JPEG crop source cannot be a graph output");
        return nullptr;
    }
    RocalTensor t = rocalJpegCOCOFileSourceSingleShard(ctx, source_path, json_path, color, shard_id, shard_count, false, shuffle, loop, p,
                                                       max_width, max_height, ROCAL_DECODER_TJPEG, si);
    if (!t) return nullptr;
    if (rb200_set_random_crop_decoder(ctx, area_factor.data(), aspect_ratio.data(), num_attempts) != ROCAL_OK) return nullptr;
    return t;
}
RocalTensor ROCAL_API_CALL rocalJpegCOCOFileSourcePartial(RocalContext ctx, const char* source_path, const char* json_path,
                                                          RocalImageColor color, unsigned internal_shard_count, bool is_output,
                                                          std::vector<float>& area_factor, std::vector<float>& aspect_ratio,
                                                          unsigned num_attempts, bool shuffle, bool loop,
                                                          RocalImageSizeEvaluationPolicy p, unsigned max_width, unsigned max_height,
                                                          RocalShardingInfo si) {
    if (internal_shard_count != 1) {
        if (ctx) P(ctx)->capture_error("rocalJpegCOCOFileSourcePartial: internal_shard_count must be 1 (use the SingleShard call per rank)");
        return nullptr;
    }
    return rocalJpegCOCOFileSourcePartialSingleShard(ctx, source_path, json_path, color, 0, 1, is_output, area_factor, aspect_ratio,
                                                     num_attempts, shuffle, loop, p, max_width, max_height, si);
}
RocalTensorList ROCAL_API_CALL rocalGetImageLabels(RocalContext ctx) {
    if (!ctx) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return nullptr;
    }
    try {
        return P(ctx)->image_label_list();
    } catch (const std::exception& e) {
        P(ctx)->capture_error(e.what());
        std::cerr << e.what() << '\n';
        return nullptr;
    }
}
void ROCAL_API_CALL rocalGetOneHotImageLabels(RocalContext ctx, void* buf, int num_classes, RocalOutputMemType m) {
    rb200_get_one_hot_image_labels(ctx, buf, num_classes, (int)m);
}
void ROCAL_API_CALL rocalGetImageSizes(RocalContext ctx, int* buf) { rb200_get_image_sizes(ctx, buf); }
void ROCAL_API_CALL rocalGetROIImageSizes(RocalContext ctx, int* buf) { rb200_get_roi_image_sizes(ctx, buf); }
void ROCAL_API_CALL rocalGetImageId(RocalContext ctx, int* buf) { rb200_get_image_ids(ctx, buf); }
unsigned ROCAL_API_CALL rocalGetImageNameLen(RocalContext ctx, int* buf) { return rb200_get_image_name_len(ctx, buf); }
void ROCAL_API_CALL rocalGetImageName(RocalContext ctx, char* buf) { rb200_get_image_name(ctx, buf); }
void ROCAL_API_CALL rocalResetLoaders(RocalContext ctx) { rb200_reset_loaders(ctx); }
size_t ROCAL_API_CALL rocalGetLastBatchPaddedSize(RocalContext ctx) { return rb200_get_last_batch_padded_size(ctx); }

RocalStatus ROCAL_API_CALL rocalExternalSourceFeedInput(RocalContext ctx, const std::vector<std::string>& input_images_names, bool,
                                                        const std::vector<unsigned char*>& input_buffer,
                                                        const std::vector<ROIxywh>& roi_xywh, unsigned int max_width,
                                                        unsigned int max_height, unsigned int channels,
                                                        RocalExternalSourceMode mode, RocalTensorLayout layout, bool eos) {
    if (mode == ROCAL_EXTSOURCE_FNAME) {
        std::vector<const char*> names;
        for (const auto& s : input_images_names) names.push_back(s.c_str());
        return (RocalStatus)rb200_feed_files(ctx, names.data(), names.size());
    }
    if (input_buffer.size() != roi_xywh.size()) {
        if (ctx) P(ctx)->capture_error("rocalExternalSourceFeedInput: one ROI per input buffer is required");
        std::cerr << "rocalExternalSourceFeedInput: one ROI per input buffer is required\n";
        return ctx ? ROCAL_RUNTIME_ERROR : ROCAL_CONTEXT_INVALID;
    }
    return (RocalStatus)rb200_feed_input(ctx, input_buffer.data(), reinterpret_cast<const unsigned*>(roi_xywh.data()),
                                         input_buffer.size(), max_width, max_height, channels, (int)mode, (int)layout, eos);
}

#define RT(x) static_cast<RocalTensor>(x)

RocalTensor ROCAL_API_CALL rocalResize(RocalContext c, RocalTensor in, unsigned dw, unsigned dh, bool out, RocalResizeScalingMode sm,
                                       std::vector<unsigned> max_size, unsigned rs, unsigned rl, RocalResizeInterpolationType it,
                                       RocalTensorLayout l, RocalTensorOutputType t) {
    if (max_size.size() > 2) {
        if (c) P(c)->capture_error("The length of max_size vector exceeds the image dimension.");
        return nullptr;
    }
    return RT(rb200_resize(c, in, dw, dh, out, (int)sm, max_size.empty() ? 0 : vec_at(max_size, 0),
                           max_size.empty() ? 0 : vec_at(max_size, 1), rs, rl, (int)it, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalResizeMirrorNormalize(RocalContext c, RocalTensor in, unsigned dw, unsigned dh, std::vector<float>& mean,
                                                      std::vector<float>& std_dev, bool out, RocalResizeScalingMode sm,
                                                      std::vector<unsigned> max_size, unsigned rs, unsigned rl,
                                                      RocalResizeInterpolationType it, RocalIntParam mirror, RocalTensorLayout l,
                                                      RocalTensorOutputType t) {
    return RT(rb200_resize_mirror_normalize(c, in, dw, dh, mean.data(), std_dev.data(), std::min(mean.size(), std_dev.size()), out,
                                            (int)sm, max_size.empty() ? 0 : vec_at(max_size, 0), max_size.empty() ? 0 : vec_at(max_size, 1),
                                            rs, rl, (int)it, mirror, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalRotate(RocalContext c, RocalTensor in, bool out, RocalFloatParam angle, unsigned dw, unsigned dh,
                                       RocalResizeInterpolationType it, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_rotate(c, in, out, angle, dw, dh, (int)it, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalRotateFixed(RocalContext c, RocalTensor in, float angle, bool out, unsigned dw, unsigned dh,
                                            RocalResizeInterpolationType it, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_rotate(c, in, out, rb200_create_float_parameter(angle), dw, dh, (int)it, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalBrightness(RocalContext c, RocalTensor in, bool out, RocalFloatParam a, RocalFloatParam b,
                                           RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_brightness(c, in, out, a, b, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalBrightnessFixed(RocalContext c, RocalTensor in, float a, float b, bool out, RocalTensorLayout l,
                                                RocalTensorOutputType t) {
    return RT(rb200_brightness(c, in, out, rb200_create_float_parameter(a), rb200_create_float_parameter(b), (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalContrast(RocalContext c, RocalTensor in, bool out, RocalFloatParam f, RocalFloatParam ce,
                                         RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_contrast(c, in, out, f, ce, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalContrastFixed(RocalContext c, RocalTensor in, float f, float ce, bool out, RocalTensorLayout l,
                                              RocalTensorOutputType t) {
    return RT(rb200_contrast(c, in, out, rb200_create_float_parameter(f), rb200_create_float_parameter(ce), (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalFlip(RocalContext c, RocalTensor in, bool out, RocalIntParam h, RocalIntParam v, RocalTensorLayout l,
                                     RocalTensorOutputType t) {
    return RT(rb200_flip(c, in, out, h, v, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalFlipFixed(RocalContext c, RocalTensor in, int h, int v, bool out, RocalTensorLayout l,
                                          RocalTensorOutputType t) {
    return RT(rb200_flip(c, in, out, rb200_create_int_parameter(h), rb200_create_int_parameter(v), (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalWarpAffine(RocalContext c, RocalTensor in, bool out, unsigned dh, unsigned dw, RocalFloatParam x0,
                                           RocalFloatParam x1, RocalFloatParam y0, RocalFloatParam y1, RocalFloatParam o0,
                                           RocalFloatParam o1, RocalResizeInterpolationType it, RocalTensorLayout l,
                                           RocalTensorOutputType t) {
    return RT(rb200_warp_affine(c, in, out, dh, dw, x0, x1, y0, y1, o0, o1, (int)it, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalWarpAffineFixed(RocalContext c, RocalTensor in, float x0, float x1, float y0, float y1, float o0, float o1,
                                                bool out, unsigned int dh, unsigned int dw, RocalResizeInterpolationType it,
                                                RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_warp_affine(c, in, out, dh, dw, rb200_create_float_parameter(x0), rb200_create_float_parameter(x1),
                                rb200_create_float_parameter(y0), rb200_create_float_parameter(y1), rb200_create_float_parameter(o0),
                                rb200_create_float_parameter(o1), (int)it, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalBlend(RocalContext c, RocalTensor in1, RocalTensor in2, bool out, RocalFloatParam r, RocalTensorLayout l,
                                      RocalTensorOutputType t) {
    return RT(rb200_blend(c, in1, in2, out, r, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalBlendFixed(RocalContext c, RocalTensor in1, RocalTensor in2, float r, bool out, RocalTensorLayout l,
                                           RocalTensorOutputType t) {
    return RT(rb200_blend(c, in1, in2, out, rb200_create_float_parameter(r), (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalGamma(RocalContext c, RocalTensor in, bool out, RocalFloatParam g, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_gamma(c, in, out, g, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalGammaFixed(RocalContext c, RocalTensor in, float g, bool out, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_gamma(c, in, out, rb200_create_float_parameter(g), (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalColorTemp(RocalContext c, RocalTensor in, bool out, RocalIntParam a, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_color_temp(c, in, out, a, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalColorTempFixed(RocalContext c, RocalTensor in, int a, bool out, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_color_temp(c, in, out, rb200_create_int_parameter(a), (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalExposure(RocalContext c, RocalTensor in, bool out, RocalFloatParam e, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_exposure(c, in, out, e, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalExposureFixed(RocalContext c, RocalTensor in, float e, bool out, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_exposure(c, in, out, rb200_create_float_parameter(e), (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalHue(RocalContext c, RocalTensor in, bool out, RocalFloatParam h, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_hue(c, in, out, h, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalHueFixed(RocalContext c, RocalTensor in, float h, bool out, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_hue(c, in, out, rb200_create_float_parameter(h), (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalSaturation(RocalContext c, RocalTensor in, bool out, RocalFloatParam s, RocalTensorLayout l,
                                           RocalTensorOutputType t) {
    return RT(rb200_saturation(c, in, out, s, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalSaturationFixed(RocalContext c, RocalTensor in, float s, bool out, RocalTensorLayout l,
                                                RocalTensorOutputType t) {
    return RT(rb200_saturation(c, in, out, rb200_create_float_parameter(s), (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalNormalize(RocalContext c, RocalTensor in, std::vector<unsigned>& axes, std::vector<float>& mean,
                                          std::vector<float>& std_dev, bool out, float scale, float shift, RocalTensorOutputType t) {
    return RT(rb200_normalize(c, in, axes.data(), (unsigned)axes.size(), mean.data(), (unsigned)mean.size(), std_dev.data(),
                              (unsigned)std_dev.size(), out, scale, shift, (int)t));
}
RocalTensor ROCAL_API_CALL rocalTranspose(RocalContext c, RocalTensor in, std::vector<unsigned> perm, bool out, RocalTensorLayout l) {
    return RT(rb200_transpose(c, in, perm.data(), (unsigned)perm.size(), out, (int)l));
}
RocalTensor ROCAL_API_CALL rocalColorTwist(RocalContext c, RocalTensor in, bool out, RocalFloatParam a, RocalFloatParam b, RocalFloatParam h,
                                           RocalFloatParam s, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_color_twist(c, in, out, a, b, h, s, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalColorTwistFixed(RocalContext c, RocalTensor in, float a, float b, float h, float s, bool out,
                                                RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_color_twist(c, in, out, rb200_create_float_parameter(a), rb200_create_float_parameter(b),
                                rb200_create_float_parameter(h), rb200_create_float_parameter(s), (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalCropMirrorNormalize(RocalContext c, RocalTensor in, unsigned ch, unsigned cw, float sx, float sy,
                                                    std::vector<float>& mean, std::vector<float>& std_dev, bool out,
                                                    RocalIntParam mirror, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_crop_mirror_normalize(c, in, ch, cw, sx, sy, mean.data(), std_dev.data(), std::min(mean.size(), std_dev.size()), out,
                                          mirror, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalCrop(RocalContext c, RocalTensor in, bool out, RocalFloatParam cw, RocalFloatParam ch, RocalFloatParam,
                                     RocalFloatParam px, RocalFloatParam py, RocalFloatParam, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_crop(c, in, out, cw, ch, px, py, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalCopy(RocalContext c, RocalTensor in, bool out) {
    return RT(rb200_flip(c, in, out, rb200_create_int_parameter(0), rb200_create_int_parameter(0), (int)ROCAL_NONE, (int)ROCAL_UINT8));
}
RocalTensor ROCAL_API_CALL rocalNop(RocalContext c, RocalTensor in, bool out) { return rocalCopy(c, in, out); }
RocalTensor ROCAL_API_CALL rocalCropResize(RocalContext c, RocalTensor in, unsigned dw, unsigned dh, bool out, RocalFloatParam area,
                                           RocalFloatParam aspect, RocalFloatParam xd, RocalFloatParam yd, RocalTensorLayout l,
                                           RocalTensorOutputType t) {
    return RT(rb200_crop_resize(c, in, dw, dh, out, area, aspect, xd, yd, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalCropResizeFixed(RocalContext c, RocalTensor in, unsigned dw, unsigned dh, bool out, float area,
                                                float aspect, float xd, float yd, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_crop_resize_fixed(c, in, dw, dh, out, area, aspect, xd, yd, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalROIResize(RocalContext c, RocalTensor in, unsigned dw, unsigned dh, bool out, unsigned roi_h,
                                          unsigned roi_w, float px, float py, RocalResizeInterpolationType interp, RocalTensorLayout l,
                                          RocalTensorOutputType t) {
    return RT(rb200_roi_resize(c, in, dw, dh, out, roi_h, roi_w, px, py, (int)interp, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalRandomCrop(RocalContext c, RocalTensor in, bool out, RocalFloatParam area, RocalFloatParam aspect,
                                           RocalFloatParam px, RocalFloatParam py, int attempts, RocalTensorLayout l,
                                           RocalTensorOutputType t) {
    return RT(rb200_random_crop(c, in, out, area, aspect, px, py, attempts, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalCropFixed(RocalContext c, RocalTensor in, unsigned cw, unsigned ch, unsigned cd, bool out, float px, float py,
                                          float, RocalTensorLayout l, RocalTensorOutputType t) {
    if (cd == 0) {
        if (c) P(c)->capture_error("Crop node needs to receive non-zero destination dimensions");
        return nullptr;
    }
    return RT(rb200_crop_fixed(c, in, cw, ch, out, px, py, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalCropCenterFixed(RocalContext c, RocalTensor in, unsigned cw, unsigned ch, unsigned cd, bool out,
                                                RocalTensorLayout l, RocalTensorOutputType t) {
    if (cd == 0) {
        if (c) P(c)->capture_error("Crop node needs to receive non-zero destination dimensions");
        return nullptr;
    }
    return RT(rb200_crop_center_fixed(c, in, cw, ch, out, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalResizeCropMirrorFixed(RocalContext c, RocalTensor in, unsigned dw, unsigned dh, bool out, unsigned crop_h,
                                                      unsigned crop_w, RocalIntParam mirror, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_resize_crop_mirror_fixed(c, in, dw, dh, out, crop_h, crop_w, mirror, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalResizeCropMirror(RocalContext c, RocalTensor in, unsigned dw, unsigned dh, bool out, RocalFloatParam crop_h,
                                                 RocalFloatParam crop_w, RocalIntParam mirror, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_resize_crop_mirror(c, in, dw, dh, out, crop_h, crop_w, mirror, (int)l, (int)t));
}
RocalTensor ROCAL_API_CALL rocalSSDRandomCrop(RocalContext c, RocalTensor in, bool out, RocalFloatParam, RocalFloatParam, RocalFloatParam,
                                              RocalFloatParam, RocalFloatParam, int attempts, RocalTensorLayout l, RocalTensorOutputType t) {
    return RT(rb200_ssd_random_crop(c, in, out, attempts, (int)l, (int)t));
}

RocalStatus ROCAL_API_CALL rocalCopyToOutput(RocalContext c, unsigned char* out_ptr, size_t out_size) {
    if (!c) return ROCAL_CONTEXT_INVALID;
    try {
        size_t off = 0;
        auto* outs = P(c)->outputs();
        for (size_t i = 0; i < outs->size(); i++) {
            rocalTensor* t = outs->at(i);
            if (off + t->data_size() > out_size) RB200_THROW("rocalCopyToOutput: the output buffer is too small");
            if (t->copy_data(out_ptr + off, ROCAL_MEMCPY_HOST)) RB200_THROW("rocalCopyToOutput: copy failed");
            off += t->data_size();
        }
    } catch (const std::exception& e) {
        P(c)->capture_error(e.what());
        std::cerr << e.what() << '\n';
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}
RocalStatus ROCAL_API_CALL rocalToTensor(RocalContext c, void* out_ptr, RocalTensorLayout fmt, RocalTensorOutputType type, float m0, float m1,
                                         float m2, float o0, float o1, float o2, bool reverse, RocalOutputMemType mem, int, int) {
    float m[3] = {m0, m1, m2}, o[3] = {o0, o1, o2};
    return (RocalStatus)rb200_to_tensor(c, out_ptr, (int)fmt, (int)type, m, o, reverse, (int)mem);
}
void ROCAL_API_CALL rocalSetOutputs(RocalContext c, unsigned int num, std::vector<RocalTensor>& outs) {
    if (!c) return;
    std::vector<rb200_tensor> v;
    for (unsigned i = 0; i < num && i < outs.size(); i++) v.push_back(outs[i]);
    rb200_set_outputs(c, v.data(), v.size());
}
RocalTensorList ROCAL_API_CALL rocalGetOutputTensors(RocalContext c) {
    if (!c) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return nullptr;
    }
    return P(c)->outputs();
}

void ROCAL_API_CALL rocalRandomBBoxCrop(RocalContext c, bool all_boxes_overlap, bool, RocalFloatParam, bool has_shape, int, int, int,
                                        RocalFloatParam, int, int64_t seed) {
    if (!c) return;
    rb200_random_bbox_crop(c, all_boxes_overlap, has_shape, (unsigned)seed);
}

void ROCAL_API_CALL rocalBoxEncoder(RocalContext c, std::vector<float>& anchors, float criteria, std::vector<float>& means,
                                    std::vector<float>& stds, bool offset, float scale) {
    if (!c) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return;
    }
    if (anchors.size() % 4 != 0 || means.size() != 4 || stds.size() != 4) {
        P(c)->capture_error("rocalBoxEncoder: anchors must hold 4 values per box; means and stds 4 values");
        return;
    }
    rb200_box_encoder(c, anchors.data(), anchors.size() / 4, criteria, means.data(), stds.data(), offset, scale);
}
void ROCAL_API_CALL rocalCopyEncodedBoxesAndLables(RocalContext c, float* boxes_buf, int* labels_buf) {
    rb200_copy_encoded_boxes_and_labels(c, boxes_buf, labels_buf);
}
RocalMetaData ROCAL_API_CALL rocalGetEncodedBoxesAndLables(RocalContext c, int num_encoded_boxes) {
    (void)num_encoded_boxes;
    if (!c) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return nullptr;
    }
    return P(c)->encoded_meta();
}

unsigned ROCAL_API_CALL rocalGetBoundingBoxCount(RocalContext c) {
    if (!c) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return 0;
    }
    try {
        return P(c)->bounding_box_count();
    } catch (const std::exception& e) {
        P(c)->capture_error(e.what());
        return 0;
    }
}
RocalTensorList ROCAL_API_CALL rocalGetBoundingBoxCords(RocalContext c) {
    if (!c) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return nullptr;
    }
    return P(c)->bounding_box_cords();
}
RocalTensorList ROCAL_API_CALL rocalGetBoundingBoxLabel(RocalContext c) {
    if (!c) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return nullptr;
    }
    return P(c)->bounding_box_labels();
}

void ROCAL_API_CALL rocalBoxIouMatcher(RocalContext c, std::vector<float>& anchors, float high_threshold, float low_threshold,
                                       bool allow_low_quality_matches) {
    if (!c) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return;
    }
    if (anchors.empty() || anchors.size() % 4 != 0) {
        P(c)->capture_error("rocalBoxIouMatcher: anchors must hold 4 values per box");
        return;
    }
    rb200_box_iou_matcher(c, anchors.data(), anchors.size() / 4, high_threshold, low_threshold, allow_low_quality_matches);
}
RocalTensorList ROCAL_API_CALL rocalGetMatchedIndices(RocalContext c) {
    if (!c) {
        std::cerr << "[ERR] Invalid rocal context\n";
        return nullptr;
    }
    return P(c)->matched_indices();
}

int ROCAL_API_CALL rocalGetOutputWidth(RocalContext c) {
    if (!c || P(c)->outputs()->size() == 0) return 0;
    return static_cast<TensorImpl*>(P(c)->outputs()->at(0))->max_w;
}
int ROCAL_API_CALL rocalGetOutputHeight(RocalContext c) {
    if (!c || P(c)->outputs()->size() == 0) return 0;
    return static_cast<TensorImpl*>(P(c)->outputs()->at(0))->max_h;
}
int ROCAL_API_CALL rocalGetOutputColorFormat(RocalContext c) { return c ? (int)ROCAL_COLOR_RGB24 : -1; }
size_t ROCAL_API_CALL rocalGetRemainingImages(RocalContext c) { return rb200_get_remaining_images(c); }
size_t ROCAL_API_CALL rocalIsEmpty(RocalContext c) { return rb200_get_remaining_images(c) == 0; }
size_t ROCAL_API_CALL rocalGetAugmentationBranchCount(RocalContext c) { return c ? (size_t)P(c)->outputs()->size() : 0; }
RocalStatus ROCAL_API_CALL rocalGetStatus(RocalContext c) { return (RocalStatus)rb200_get_status(c); }
const char* ROCAL_API_CALL rocalGetErrorMessage(RocalContext c) { return rb200_get_error_message(c); }
TimingInfo ROCAL_API_CALL rocalGetTimingInfo(RocalContext c) {
    TimingInfo t{0, 0, 0, 0};
    if (c) t = P(c)->timing();
    return t;
}

}  // extern "C"
