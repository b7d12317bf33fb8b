// Plain C ABI of the pipeline (include/rb200.h). Every entry point validates its handles, runs the
// call inside try/catch, stores a failure in the context and prints it to stderr — the error
// convention of the reference's API layer (rocAL/include/api/rocal_api.h:42-62,
// rocAL/include/pipeline/context.h:41-51).
#include <cstdio>
#include <cstring>
#include <iostream>

#include "pipeline.h"

using namespace rb200;

namespace {

inline Pipeline* P(rb200_context c) { return static_cast<Pipeline*>(c); }
inline TensorImpl* T(rb200_tensor t) { return static_cast<TensorImpl*>(static_cast<rocalTensor*>(t)); }
inline IntParam* IP(rb200_param p) { return static_cast<IntParam*>(p); }
inline FloatParam* FP(rb200_param p) { return static_cast<FloatParam*>(p); }

void report(Pipeline* p, const std::exception& e) {
    p->capture_error(e.what());
    if (rb200::log_level() >= 1) std::cerr << e.what() << '\n';
}

#define CTX_OR(ret)                                        \
    if (ctx == nullptr) {                                  \
        std::cerr << "[ERR] Invalid rocal context\n";      \
        return ret;                                        \
    }
#define IN_OR_NULL                                         \
    if (in == nullptr) {                                   \
        std::cerr << "[ERR] Invalid input image\n";        \
        return nullptr;                                    \
    }

Parameter<int>* int_param(rb200_param p, int lo, int hi) {
    return p ? IP(p)->core : ParameterFactory::instance().default_uniform_int(lo, hi);
}
Parameter<float>* float_param(rb200_param p, float lo, float hi) {
    return p ? FP(p)->core : ParameterFactory::instance().default_uniform_float(lo, hi);
}

// The normalisation tables of CropMirrorNormalizeNode::create_node (node_crop_mirror_normalize.cpp:46-70):
// 1/std and -(mean * (1/std)) per channel.
void set_normalize(Node& nd, const float* mean, const float* std_dev, size_t n) {
    if (!mean || !std_dev || n == 0) RB200_THROW("Mean or std dev array is empty");
    for (int c = 0; c < 3; c++) {
        float m = mean[n >= 3 ? c : 0], s = std_dev[n >= 3 ? c : 0];
        if (!s) RB200_THROW("Standard deviation value cannot be 0");
        float inv = 1 / s;
        nd.mul[c] = inv;
        nd.add[c] = -(m * inv);
    }
    nd.normalize = true;
}

// Output shape rules of rocalResize / rocalResizeMirrorNormalize (source/api/rocal_api_augmentation.cpp:449-506,
// 550-621). allow_min_max: only ResizeMirrorNormalize knows ROCAL_SCALING_MODE_MIN_MAX, where resize_shorter and
// resize_longer carry the minimum and maximum size and travel to the node in place of max_size.
void resize_shapes(TensorImpl* in, unsigned dest_w, unsigned dest_h, int scaling_mode, unsigned max_w, unsigned max_h,
                   unsigned resize_shorter, unsigned resize_longer, Node& nd, unsigned& out_max_w, unsigned& out_max_h,
                   bool allow_min_max = false) {
    const unsigned kMaxAspectRatio = 6;   // MAX_ASPECT_RATIO, include/pipeline/commons.h:39
    const bool min_max = scaling_mode == ROCAL_SCALING_MODE_MIN_MAX;
    if (min_max && !allow_min_max) RB200_THROW("ROCAL_SCALING_MODE_MIN_MAX is a mode of rocalResizeMirrorNormalize only");
    if ((dest_w | dest_h | resize_longer | resize_shorter) == 0)
        RB200_THROW("Atleast one size 'dest_width' or 'dest_height' or 'resize_shorter' or 'resize_longer' must be specified");
    if ((dest_w | dest_h) && (resize_longer | resize_shorter) && !min_max)
        RB200_THROW("Only one method of specifying size can be used \ndest_width and/or dest_height\nresize_shorter\nresize_longer");
    if (resize_longer && resize_shorter && !min_max)
        RB200_THROW("'resize_longer' and 'resize_shorter' cannot be passed together. They are mutually exclusive.");
    if (min_max && (!resize_shorter || !resize_longer))
        RB200_THROW("ROCAL_SCALING_MODE_MIN_MAX needs the minimum size in resize_shorter and the maximum size in resize_longer");
    unsigned out_w, out_h;
    int mode;
    if (min_max) {
        mode = scaling_mode;
        out_w = dest_w;
        out_h = dest_h;
    } else if (resize_shorter) {
        mode = ROCAL_SCALING_MODE_NOT_SMALLER;
        out_w = out_h = resize_shorter;
    } else if (resize_longer) {
        mode = ROCAL_SCALING_MODE_NOT_LARGER;
        out_w = out_h = resize_longer;
    } else {
        mode = scaling_mode;
        out_w = dest_w;
        out_h = dest_h;
    }
    if (max_w != 0 && max_h != 0) {
        out_max_w = max_w;
        out_max_h = max_h;
    } else {
        if (mode == ROCAL_SCALING_MODE_STRETCH) {
            out_max_w = out_w ? out_w : (unsigned)in->max_w;
            out_max_h = out_h ? out_h : (unsigned)in->max_h;
        } else if (mode == ROCAL_SCALING_MODE_NOT_SMALLER) {
            out_max_w = (out_w ? out_w : out_h) * kMaxAspectRatio;
            out_max_h = (out_h ? out_h : out_w) * kMaxAspectRatio;
        } else {
            out_max_w = out_w ? out_w : out_h * kMaxAspectRatio;
            out_max_h = out_h ? out_h : out_w * kMaxAspectRatio;
        }
        if (max_w) out_max_w = max_w;
        if (max_h) out_max_h = max_h;
    }
    if (min_max && (out_max_w == 0 || out_max_h == 0)) {
        // neither dest sizes nor max_size were given: the longer side never exceeds the maximum size
        out_max_w = out_max_h = resize_longer;
    }
    nd.dest_w = out_w;
    nd.dest_h = out_h;
    nd.scaling_mode = mode;
    nd.max_w = min_max ? resize_shorter : max_w;
    nd.max_h = min_max ? resize_longer : max_h;
}

// Resize-type operators take every filter of RocalResizeInterpolationType (rocal_api_types.h:347-367).
int resize_interpolation(int interpolation) {
    switch (interpolation) {
        case ROCAL_LINEAR_INTERPOLATION: return RB200_INTERP_BILINEAR;
        case ROCAL_TRIANGULAR_INTERPOLATION: return RB200_INTERP_TRIANGULAR;
        case ROCAL_CUBIC_INTERPOLATION: return RB200_INTERP_BICUBIC;
        case ROCAL_LANCZOS_INTERPOLATION: return RB200_INTERP_LANCZOS;
        case ROCAL_GAUSSIAN_INTERPOLATION: return RB200_INTERP_GAUSSIAN;
        case ROCAL_NEAREST_NEIGHBOR_INTERPOLATION: return RB200_INTERP_NEAREST;
        default: RB200_THROW("unknown interpolation type " + std::to_string(interpolation));
    }
}

void check_interpolation(int interpolation) {
    if (interpolation != ROCAL_LINEAR_INTERPOLATION)
        RB200_THROW("only ROCAL_LINEAR_INTERPOLATION is implemented for this operator");
}

rb200_tensor finish(Pipeline* p, Node&& nd, TensorImpl* in, unsigned w, unsigned h, int lay, int dt, int is_output) {
    return static_cast<rocalTensor*>(
        p->add_node(std::move(nd), in, w, h, (RocalTensorLayout)lay, (RocalTensorOutputType)dt, is_output != 0));
}

// ---- DLPack (v0 ABI) ----
struct DLDevice { int32_t device_type; int32_t device_id; };
struct DLDataType { uint8_t code; uint8_t bits; uint16_t lanes; };
struct DLTensor { void* data; DLDevice device; int32_t ndim; DLDataType dtype; int64_t* shape; int64_t* strides; uint64_t byte_offset; };
struct DLManagedTensor { DLTensor dl_tensor; void* manager_ctx; void (*deleter)(DLManagedTensor*); };
void dl_deleter(DLManagedTensor* m) {
    if (!m) return;
    delete[] m->dl_tensor.shape;
    delete[] m->dl_tensor.strides;
    delete m;
}

}  // namespace

extern "C" {

rb200_context rb200_create(size_t batch_size, int affinity, int gpu_id, size_t cpu_thread_count,
                           size_t prefetch_queue_depth, int output_tensor_data_type) {
    (void)cpu_thread_count;
    try {
        if (affinity != ROCAL_PROCESS_GPU)
            RB200_THROW("this library has no CPU backend: create the context with ROCAL_PROCESS_GPU");
        auto* p = new Pipeline(batch_size, gpu_id, prefetch_queue_depth, (RocalTensorOutputType)output_tensor_data_type);
        // MasterGraph's constructor seeds the parameter factory with 0 (master_graph.cpp:186).
        ParameterFactory::instance().set_seed(0);
        return p;
    } catch (const std::exception& e) {
        std::cerr << "rocalCreate: " << e.what() << '\n';
        return nullptr;
    }
}

int rb200_verify(rb200_context ctx) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        P(ctx)->verify();
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_run(rb200_context ctx) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        P(ctx)->run();
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_release(rb200_context ctx) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        delete P(ctx);
    } catch (const std::exception& e) {
        std::cerr << e.what() << '\n';
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_get_status(rb200_context ctx) {
    if (!ctx) return ROCAL_CONTEXT_INVALID;
    return P(ctx)->status();
}
const char* rb200_get_error_message(rb200_context ctx) {
    if (!ctx) return "Invalid rocal context";
    return P(ctx)->error_message();
}
void rb200_get_timing(rb200_context ctx, unsigned long long out[4]) {
    out[0] = out[1] = out[2] = out[3] = 0;
    if (!ctx) return;
    TimingInfo t = P(ctx)->timing();
    out[0] = t.load_time; out[1] = t.decode_time; out[2] = t.process_time; out[3] = t.transfer_time;
}
size_t rb200_get_remaining_images(rb200_context ctx) { return ctx ? P(ctx)->remaining() : 0; }
unsigned long long rb200_get_h2d_bytes(rb200_context ctx) { return ctx ? P(ctx)->h2d_bytes() : 0; }
int rb200_set_upload_mode(rb200_context ctx, int mode) {
    if (!ctx || mode < 0 || mode > 2) return -1;
    P(ctx)->set_upload_mode(mode);
    return 0;
}

int rb200_set_arithmetic(rb200_context ctx, int mode) {
    if (!ctx) return -1;
    try {
        P(ctx)->set_arithmetic(mode);
        return 0;
    } catch (const std::exception& e) {
        P(ctx)->capture_error(e.what());
        return -1;
    }
}
int rb200_consumer_fence(rb200_context ctx, void* cuda_stream) {
    if (!ctx) return -1;
    try {
        P(ctx)->consumer_fence(cuda_stream);
        return 0;
    } catch (const std::exception& e) {
        P(ctx)->capture_error(e.what());
        return -1;
    }
}
int rb200_set_wait_probe(rb200_context ctx, unsigned long long wait_cycles, int skip_row) {
    if (!ctx) return -1;
    P(ctx)->set_wait_probe(wait_cycles, skip_row);
    return 0;
}

// ---- parameters ----
void rb200_set_seed(unsigned seed) { ParameterFactory::instance().set_seed(seed); }
unsigned rb200_get_seed(void) { return ParameterFactory::instance().get_seed(); }
rb200_param rb200_create_int_uniform_rand(int start, int end) { return ParameterFactory::instance().create_uniform_int(start, end); }
rb200_param rb200_create_float_uniform_rand(float start, float end) { return ParameterFactory::instance().create_uniform_float(start, end); }
rb200_param rb200_create_int_rand(const int* values, const double* frequencies, unsigned size) {
    if (!values || !frequencies || size == 0) return nullptr;
    return ParameterFactory::instance().create_custom_int(values, frequencies, size);
}
rb200_param rb200_create_float_rand(const float* values, const double* frequencies, unsigned size) {
    if (!values || !frequencies || size == 0) return nullptr;
    return ParameterFactory::instance().create_custom_float(values, frequencies, size);
}
rb200_param rb200_create_int_parameter(int value) { return ParameterFactory::instance().create_int(value); }
rb200_param rb200_create_float_parameter(float value) { return ParameterFactory::instance().create_float(value); }
int rb200_update_int_parameter(int value, rb200_param p) {
    if (!p || !ParameterFactory::instance().owns(p)) return ROCAL_UPDATE_PARAMETER_FAILED;
    if (IP(p)->kind != ParamKind::DETERMINISTIC) return ROCAL_INVALID_PARAMETER_TYPE;
    static_cast<SimpleParameter<int>*>(IP(p)->core)->update(value);
    return ROCAL_OK;
}
int rb200_update_float_parameter(float value, rb200_param p) {
    if (!p || !ParameterFactory::instance().owns(p)) return ROCAL_UPDATE_PARAMETER_FAILED;
    if (FP(p)->kind != ParamKind::DETERMINISTIC) return ROCAL_INVALID_PARAMETER_TYPE;
    static_cast<SimpleParameter<float>*>(FP(p)->core)->update(value);
    return ROCAL_OK;
}
int rb200_update_int_uniform_rand(int start, int end, rb200_param p) {
    if (!p || !ParameterFactory::instance().owns(p)) return ROCAL_UPDATE_PARAMETER_FAILED;
    if (IP(p)->kind != ParamKind::RANDOM_UNIFORM) return ROCAL_INVALID_PARAMETER_TYPE;
    static_cast<UniformRand<int>*>(IP(p)->core)->update(start, end);
    return ROCAL_OK;
}
int rb200_update_float_uniform_rand(float start, float end, rb200_param p) {
    if (!p || !ParameterFactory::instance().owns(p)) return ROCAL_UPDATE_PARAMETER_FAILED;
    if (FP(p)->kind != ParamKind::RANDOM_UNIFORM) return ROCAL_INVALID_PARAMETER_TYPE;
    static_cast<UniformRand<float>*>(FP(p)->core)->update(start, end);
    return ROCAL_OK;
}
int rb200_get_int_value(rb200_param p) { return p ? IP(p)->core->get() : 0; }
float rb200_get_float_value(rb200_param p) { return p ? FP(p)->core->get() : 0.f; }

// ---- input ----
rb200_tensor rb200_external_source(rb200_context ctx, int color_format, int is_output, unsigned max_width,
                                   unsigned max_height, int external_source_mode) {
    CTX_OR(nullptr);
    try {
        if (external_source_mode != ROCAL_EXTSOURCE_RAW_UNCOMPRESSED && external_source_mode != ROCAL_EXTSOURCE_RAW_COMPRESSED &&
            external_source_mode != ROCAL_EXTSOURCE_FNAME)
            RB200_THROW("bad external source mode");
        if (color_format != ROCAL_COLOR_RGB24 && color_format != ROCAL_COLOR_BGR24)
            RB200_THROW("only 3-channel interleaved colour formats are supported");
        return static_cast<rocalTensor*>(P(ctx)->add_source(max_width, max_height, is_output != 0));
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return nullptr;
    }
}

int rb200_feed_input(rb200_context ctx, const unsigned char* const* buffers, const unsigned* roi_xywh, size_t n,
                     unsigned max_width, unsigned max_height, unsigned channels, int mode, int layout, int eos) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    (void)eos;
    try {
        if (mode == ROCAL_EXTSOURCE_RAW_COMPRESSED) {
            // JPEG streams; the byte length of buffer i travels in roi[i].h
            // (rocAL/source/loaders/image/image_read_and_decode.cpp:123-124)
            if (!buffers || !roi_xywh) RB200_THROW("null input buffers or ROI");
            InputBatch b;
            b.kind = InputBatch::ENCODED;
            b.n = n;
            b.bufs.assign(buffers, buffers + n);
            b.enc_sizes.resize(n);
            for (size_t i = 0; i < n; i++) b.enc_sizes[i] = roi_xywh[i * 4 + 3];
            P(ctx)->feed(std::move(b));
            return ROCAL_OK;
        }
        if (mode != ROCAL_EXTSOURCE_RAW_UNCOMPRESSED)
            RB200_THROW("rb200_feed_input takes RAW_UNCOMPRESSED or RAW_COMPRESSED buffers; file names go through rb200_feed_files");
        if (channels != 3) RB200_THROW("only 3-channel input is supported");
        if (layout != ROCAL_NHWC) RB200_THROW("raw input must be NHWC");
        if (!buffers || !roi_xywh) RB200_THROW("null input buffers or ROI");
        InputBatch b;
        b.kind = InputBatch::SLOTS;
        b.n = n;
        b.bufs.assign(buffers, buffers + n);
        b.roi.assign(roi_xywh, roi_xywh + n * 4);
        b.max_w = max_width;
        b.max_h = max_height;
        P(ctx)->feed(std::move(b));
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_feed_encoded(rb200_context ctx, const unsigned char* const* buffers, const size_t* sizes, size_t n) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!buffers || !sizes) RB200_THROW("null input buffers or sizes");
        InputBatch b;
        b.kind = InputBatch::ENCODED;
        b.n = n;
        b.bufs.assign(buffers, buffers + n);
        b.enc_sizes.assign(sizes, sizes + n);
        P(ctx)->feed(std::move(b));
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_feed_files(rb200_context ctx, const char* const* paths, size_t n) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!paths) RB200_THROW("null file name list");
        InputBatch b;
        b.kind = InputBatch::ENCODED;
        b.n = n;
        for (size_t i = 0; i < n; i++) {
            if (!paths[i]) RB200_THROW("null file name");
            b.paths.emplace_back(paths[i]);
        }
        P(ctx)->feed(std::move(b));
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_set_file_list(rb200_context ctx, const char* file_list_path) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    P(ctx)->note_file_list(file_list_path ? file_list_path : "");
    return ROCAL_OK;
}

rb200_tensor rb200_jpeg_file_source(rb200_context ctx, const char* source_path, int color_format, unsigned shard_id,
                                    unsigned shard_count, int is_output, int shuffle, int loop, unsigned max_width,
                                    unsigned max_height, int last_batch_policy, int pad_last_batch_repeated) {
    CTX_OR(nullptr);
    try {
        if (!source_path) RB200_THROW("null source path");
        if (color_format != ROCAL_COLOR_RGB24) RB200_THROW("the file source decodes to ROCAL_COLOR_RGB24 only");
        return static_cast<rocalTensor*>(P(ctx)->add_file_source(source_path, shard_id, shard_count, shuffle != 0, loop != 0, max_width,
                                                                 max_height, is_output != 0, last_batch_policy,
                                                                 pad_last_batch_repeated != 0));
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return nullptr;
    }
}

rb200_tensor rb200_coco_file_source(rb200_context ctx, const char* source_path, const char* json_path, int color_format,
                                    unsigned shard_id, unsigned shard_count, int is_output, int shuffle, int loop, unsigned max_width,
                                    unsigned max_height, int last_batch_policy, int pad_last_batch_repeated, int avoid_class_remapping) {
    CTX_OR(nullptr);
    try {
        if (!source_path || !json_path) RB200_THROW("null source or annotation path");
        if (color_format != ROCAL_COLOR_RGB24) RB200_THROW("the file source decodes to ROCAL_COLOR_RGB24 only");
        return static_cast<rocalTensor*>(P(ctx)->add_coco_source(source_path, json_path, avoid_class_remapping != 0, shard_id, shard_count,
                                                                 shuffle != 0, loop != 0, max_width, max_height, is_output != 0,
                                                                 last_batch_policy, pad_last_batch_repeated != 0));
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return nullptr;
    }
}

namespace {
rb200::RandomCropRanges crop_ranges(const float* area_factor, const float* aspect_ratio, unsigned num_attempts) {
    if (!area_factor || !aspect_ratio) RB200_THROW("area_factor and aspect_ratio must point to two floats each");
    rb200::RandomCropRanges r;
    r.area_lo = area_factor[0];
    r.area_hi = area_factor[1];
    r.aspect_lo = aspect_ratio[0];
    r.aspect_hi = aspect_ratio[1];
    r.num_attempts = (int)num_attempts;
    if (!(r.area_lo > 0.f) || r.area_hi < r.area_lo || !(r.aspect_lo > 0.f) || r.aspect_hi < r.aspect_lo || r.num_attempts < 1)
        RB200_THROW("fused JPEG crop: area_factor and aspect_ratio must be positive ascending pairs, num_attempts >= 1");
    return r;
}
}  // namespace

rb200_tensor rb200_fused_jpeg_crop_file_source(rb200_context ctx, const char* source_path, int color_format, unsigned shard_id,
                                               unsigned shard_count, int is_output, const float* area_factor,
                                               const float* aspect_ratio, unsigned num_attempts, int shuffle, int loop,
                                               unsigned max_width, unsigned max_height, int last_batch_policy,
                                               int pad_last_batch_repeated) {
    CTX_OR(nullptr);
    try {
        if (!source_path) RB200_THROW("null source path");
        if (color_format != ROCAL_COLOR_RGB24) RB200_THROW("the file source decodes to ROCAL_COLOR_RGB24 only");
        if (is_output) RB200_THROW("the fused JPEG crop source cannot be a graph output");
        const rb200::RandomCropRanges r = crop_ranges(area_factor, aspect_ratio, num_attempts);
        rb200::TensorImpl* t = P(ctx)->add_file_source(source_path, shard_id, shard_count, shuffle != 0, loop != 0, max_width,
                                                       max_height, false, last_batch_policy, pad_last_batch_repeated != 0);
        P(ctx)->set_random_crop_decoder(r);
        return static_cast<rocalTensor*>(t);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return nullptr;
    }
}

int rb200_set_random_crop_decoder(rb200_context ctx, const float* area_factor, const float* aspect_ratio, unsigned num_attempts) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        P(ctx)->set_random_crop_decoder(crop_ranges(area_factor, aspect_ratio, num_attempts));
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_INVALID_PARAMETER_TYPE;
    }
    return ROCAL_OK;
}

int rb200_get_decoder_crop_windows(rb200_context ctx, unsigned* xywh, unsigned* batch_seed) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        P(ctx)->decoder_crop_windows(xywh, batch_seed);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_set_profiling(rb200_context ctx, int on) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        P(ctx)->set_profiling(on != 0);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_INVALID_PARAMETER_TYPE;
    }
    return ROCAL_OK;
}

size_t rb200_get_step_timing(rb200_context ctx, rb200_step_timing* out, size_t capacity) {
    if (ctx == nullptr) return 0;
    const std::vector<rb200::StepTiming> v = P(ctx)->step_timing();
    for (size_t i = 0; i < v.size() && i < capacity && out; i++) {
        std::memset(&out[i], 0, sizeof(out[i]));
        std::strncpy(out[i].name, v[i].name.c_str(), sizeof(out[i].name) - 1);
        out[i].gpu_us = v[i].gpu_us;
        out[i].batches = v[i].batches;
    }
    return v.size();
}

int rb200_random_bbox_crop(rb200_context ctx, int all_boxes_overlap, int has_shape, unsigned seed) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        P(ctx)->set_random_bbox_crop(all_boxes_overlap != 0, has_shape != 0, seed);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_INVALID_PARAMETER_TYPE;
    }
    return ROCAL_OK;
}

int rb200_get_bbox_crop_windows(rb200_context ctx, float* xywh) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        P(ctx)->bbox_crop_windows(xywh);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_bbox_crop_windows(unsigned seed, int all_boxes_overlap, int has_shape, const float* boxes_ltrb, const int* box_offsets,
                            size_t n, const int* img_widths, float* out_xywh) {
    try {
        if (n && (!box_offsets || !img_widths || !out_xywh)) return ROCAL_INVALID_PARAMETER_TYPE;
        rb200::BBoxCropSampler sampler(seed, all_boxes_overlap != 0, has_shape != 0);
        for (size_t i = 0; i < n; i++) {
            const int nb = box_offsets[i + 1] - box_offsets[i];
            if (nb < 0 || (nb > 0 && !boxes_ltrb) || img_widths[i] <= 0) return ROCAL_INVALID_PARAMETER_TYPE;
            sampler.window(boxes_ltrb + (size_t)box_offsets[i] * 4, nb, img_widths[i], out_xywh + i * 4);
        }
    } catch (const std::exception&) {
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_random_crop_windows(unsigned batch_seed, const int* shapes_hw, size_t n, const float* area_factor,
                              const float* aspect_ratio, unsigned num_attempts, unsigned* out_xywh) {
    try {
        if (n && (!shapes_hw || !out_xywh)) return ROCAL_INVALID_PARAMETER_TYPE;
        const rb200::RandomCropRanges r = crop_ranges(area_factor, aspect_ratio, num_attempts);
        const std::vector<uint32_t> seeds = rb200::random_crop_sample_seeds(batch_seed, n);
        for (size_t i = 0; i < n; i++) {
            const rb200::CropRect w = rb200::random_crop_window(shapes_hw[i * 2], shapes_hw[i * 2 + 1], seeds[i], r);
            out_xywh[i * 4] = w.x;
            out_xywh[i * 4 + 1] = w.y;
            out_xywh[i * 4 + 2] = w.w;
            out_xywh[i * 4 + 3] = w.h;
        }
    } catch (const std::exception&) {
        return ROCAL_INVALID_PARAMETER_TYPE;
    }
    return ROCAL_OK;
}

int rb200_reset_loaders(rb200_context ctx) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        P(ctx)->reset_loaders();
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_get_image_labels(rb200_context ctx, int* labels) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!labels) RB200_THROW("null output buffer");
        P(ctx)->image_labels(labels);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

unsigned rb200_get_image_name_len(rb200_context ctx, int* lengths) {
    if (!ctx) return 0;
    try {
        unsigned total = 0;
        const auto& names = P(ctx)->image_names();
        for (size_t i = 0; i < names.size(); i++) {
            if (lengths) lengths[i] = (int)names[i].size();
            total += (unsigned)names[i].size();
        }
        return total;
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return 0;
    }
}

int rb200_get_image_name(rb200_context ctx, char* buf) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!buf) RB200_THROW("null output buffer");
        size_t pos = 0;
        for (const auto& nm : P(ctx)->image_names()) {
            std::memcpy(buf + pos, nm.data(), nm.size());
            pos += nm.size();
        }
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

// rocalGetOneHotImageLabels (source/api/rocal_api_meta_data.cpp:229-266): label k > 0 sets position k-1, label 0
// sets the last position, anything else leaves the row at zero.
int rb200_get_one_hot_image_labels(rb200_context ctx, void* buf, int num_classes, int output_mem_type) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!buf || num_classes <= 0) RB200_THROW("null buffer or non-positive class count");
        const size_t n = (size_t)P(ctx)->batch();
        std::vector<int> labels(n);
        P(ctx)->image_labels(labels.data());
        std::vector<int> hot(n * (size_t)num_classes, 0);
        for (size_t i = 0; i < n; i++) {
            const int k = labels[i];
            if (k > 0 && k <= num_classes) hot[i * num_classes + k - 1] = 1;
            else if (k == 0) hot[i * num_classes + num_classes - 1] = 1;
        }
        if (output_mem_type == ROCAL_MEMCPY_HOST)
            std::memcpy(buf, hot.data(), hot.size() * sizeof(int));
        else
            P(ctx)->sync_copy(buf, hot.data(), hot.size() * sizeof(int), cudaMemcpyHostToDevice);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

// rocalGetImageSizes (rocal_api_meta_data.cpp:335-349): width, height of every source image of the batch.
int rb200_get_image_sizes(rb200_context ctx, int* buf) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!buf) RB200_THROW("null output buffer");
        P(ctx)->source_sizes(buf);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_get_image_ids(rb200_context ctx, int* buf) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!buf) RB200_THROW("null output buffer");
        P(ctx)->image_ids(buf);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

// rocalGetROIImageSizes (rocal_api_meta_data.cpp:353-372).
int rb200_get_roi_image_sizes(rb200_context ctx, int* buf) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!buf) RB200_THROW("null output buffer");
        P(ctx)->roi_image_sizes(buf);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

size_t rb200_get_last_batch_padded_size(rb200_context ctx) { return ctx ? P(ctx)->last_batch_padded_size() : 0; }

int rb200_feed_ragged(rb200_context ctx, const void* arena, size_t arena_bytes, const rb200_image_desc* descs, size_t n,
                      int mem_kind) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!descs) RB200_THROW("null image descriptors");
        if (mem_kind < RB200_MEM_HOST || mem_kind > RB200_MEM_DEVICE) RB200_THROW("bad mem_kind");
        InputBatch b;
        b.kind = InputBatch::RAGGED;
        b.n = n;
        b.arena = arena;
        b.arena_bytes = arena_bytes;
        b.mem_kind = mem_kind;
        b.descs.assign(descs, descs + n);
        P(ctx)->feed(std::move(b));
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_feed_boxes(rb200_context ctx, const float* ltrb, const int* labels, const int* counts, size_t n) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!ltrb || !labels || !counts) RB200_THROW("null box arrays");
        P(ctx)->stage_boxes(ltrb, labels, counts, n);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_set_crop_anchors(rb200_context ctx, rb200_tensor t, const float* ax, const float* ay, size_t n) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!t || !ax || !ay) RB200_THROW("null argument");
        P(ctx)->stage_anchors(T(t), ax, ay, n);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_set_affine(rb200_context ctx, rb200_tensor t, const float* m6, size_t n) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!t || !m6) RB200_THROW("null argument");
        P(ctx)->stage_affine(T(t), m6, n);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

// ---- augmentations ----
#define API_BEGIN     \
    CTX_OR(nullptr);  \
    IN_OR_NULL;       \
    Pipeline* p = P(ctx); \
    try {
#define API_END                        \
    }                                  \
    catch (const std::exception& e) {  \
        report(p, e);                  \
        return nullptr;                \
    }

rb200_tensor rb200_resize(rb200_context ctx, rb200_tensor in, unsigned dest_width, unsigned dest_height, int is_output,
                          int scaling_mode, unsigned max_w, unsigned max_h, unsigned resize_shorter,
                          unsigned resize_longer, int interpolation, int out_layout, int out_dtype) {
    API_BEGIN
    Node nd;
    nd.interpolation = resize_interpolation(interpolation);
    nd.kind = NodeKind::RESIZE;
    unsigned mw, mh;
    resize_shapes(T(in), dest_width, dest_height, scaling_mode, max_w, max_h, resize_shorter, resize_longer, nd, mw, mh);
    return finish(p, std::move(nd), T(in), mw, mh, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_resize_mirror_normalize(rb200_context ctx, rb200_tensor in, unsigned dest_width, unsigned dest_height,
                                           const float* mean, const float* std_dev, size_t n_mean, int is_output,
                                           int scaling_mode, unsigned max_w, unsigned max_h, unsigned resize_shorter,
                                           unsigned resize_longer, int interpolation, rb200_param mirror, int out_layout,
                                           int out_dtype) {
    API_BEGIN
    Node nd;
    nd.interpolation = resize_interpolation(interpolation);
    nd.kind = NodeKind::RESIZE_MIRROR_NORMALIZE;
    unsigned mw, mh;
    resize_shapes(T(in), dest_width, dest_height, scaling_mode, max_w, max_h, resize_shorter, resize_longer, nd, mw, mh, true);
    set_normalize(nd, mean, std_dev, n_mean);
    nd.mirror = int_param(mirror, 0, 1);
    return finish(p, std::move(nd), T(in), mw, mh, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_crop_mirror_normalize(rb200_context ctx, rb200_tensor in, unsigned crop_height, unsigned crop_width,
                                         float start_x, float start_y, const float* mean, const float* std_dev,
                                         size_t n_mean, int is_output, rb200_param mirror, int out_layout, int out_dtype) {
    API_BEGIN
    if (crop_width == 0 || crop_height == 0) RB200_THROW("Null values passed as input");
    Node nd;
    nd.kind = NodeKind::CROP_MIRROR_NORMALIZE;
    nd.crop.mode = CropSpec::FIXED_ANCHOR;
    nd.crop.crop_w = crop_width;
    nd.crop.crop_h = crop_height;
    nd.crop.anchor_x = start_x;
    nd.crop.anchor_y = start_y;
    set_normalize(nd, mean, std_dev, n_mean);
    nd.mirror = int_param(mirror, 0, 1);
    return finish(p, std::move(nd), T(in), crop_width, crop_height, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_crop(rb200_context ctx, rb200_tensor in, int is_output, rb200_param crop_width, rb200_param crop_height,
                        rb200_param crop_pos_x, rb200_param crop_pos_y, int out_layout, int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::CROP;
    nd.crop.mode = CropSpec::RANDOM;
    nd.crop.w_factor = float_param(crop_width, 0.55f, 0.95f);
    nd.crop.h_factor = float_param(crop_height, 0.55f, 0.95f);
    nd.crop.x_drift = float_param(crop_pos_x, 0.01f, 0.99f);
    nd.crop.y_drift = float_param(crop_pos_y, 0.01f, 0.99f);
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

namespace {
// The random-area window of RocalRandomCropParam as an internal crop node in front of `consumer`.
// Null handles become the class's default ranges, created in the class's order from the seed table
// (include/parameters/parameter_crop.h:48-51, parameter_random_crop.h:30-33,42-43).
Parameter<float>* table_float_param(rb200_param p, float lo, float hi) {
    return p ? FP(p)->core : ParameterFactory::instance().create_uniform_float(lo, hi)->core;
}
void set_random_area(CropSpec& crop, rb200_param area, rb200_param aspect, rb200_param x_drift, rb200_param y_drift) {
    crop.mode = CropSpec::RANDOM_AREA;
    crop.x_drift = table_float_param(x_drift, 0.01f, 0.99f);
    crop.y_drift = table_float_param(y_drift, 0.01f, 0.99f);
    crop.area = table_float_param(area, 0.08f, 0.99f);
    crop.aspect = table_float_param(aspect, 0.7500f, 1.333f);
}
}  // namespace

rb200_tensor rb200_random_crop(rb200_context ctx, rb200_tensor in, int is_output, rb200_param crop_area_factor,
                               rb200_param crop_aspect_ratio, rb200_param crop_pos_x, rb200_param crop_pos_y, int num_of_attempts,
                               int out_layout, int out_dtype) {
    API_BEGIN
    (void)num_of_attempts;   // the reference's window rule always makes five attempts (parameter_random_crop.cpp:52)
    Node nd;
    nd.kind = NodeKind::CROP;
    set_random_area(nd.crop, crop_area_factor, crop_aspect_ratio, crop_pos_x, crop_pos_y);
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

int rb200_random_area_windows(const unsigned* wh, size_t n, rb200_param area, rb200_param aspect_ratio, rb200_param x_drift,
                              rb200_param y_drift, unsigned* out_xywh) {
    try {
        if (n && (!wh || !out_xywh)) return ROCAL_INVALID_PARAMETER_TYPE;
        CropSpec crop;
        set_random_area(crop, area, aspect_ratio, x_drift, y_drift);
        std::vector<int> w(n), h(n);
        for (size_t i = 0; i < n; i++) {
            w[i] = (int)wh[i * 2];
            h[i] = (int)wh[i * 2 + 1];
        }
        crop.update(w, h);
        for (size_t i = 0; i < n; i++) {
            out_xywh[i * 4] = crop.x1v[i];
            out_xywh[i * 4 + 1] = crop.y1v[i];
            out_xywh[i * 4 + 2] = crop.cwv[i];
            out_xywh[i * 4 + 3] = crop.chv[i];
        }
    } catch (const std::exception&) {
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

rb200_tensor rb200_crop_resize(rb200_context ctx, rb200_tensor in, unsigned dest_width, unsigned dest_height, int is_output,
                               rb200_param area, rb200_param aspect_ratio, rb200_param x_center_drift, rb200_param y_center_drift,
                               int out_layout, int out_dtype) {
    API_BEGIN
    if (dest_width == 0 || dest_height == 0) RB200_THROW("CropResize node needs tp receive non-zero destination dimensions");
    Node window;
    window.kind = NodeKind::CROP;
    set_random_area(window.crop, area, aspect_ratio, x_center_drift, y_center_drift);
    TensorImpl* cut = p->add_node(std::move(window), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, ROCAL_NHWC, ROCAL_UINT8, false);
    Node nd;
    nd.kind = NodeKind::RESIZE;
    nd.dest_w = dest_width;
    nd.dest_h = dest_height;
    nd.scaling_mode = ROCAL_SCALING_MODE_STRETCH;
    return finish(p, std::move(nd), cut, dest_width, dest_height, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_crop_resize_fixed(rb200_context ctx, rb200_tensor in, unsigned dest_width, unsigned dest_height, int is_output,
                                     float area, float aspect_ratio, float x_center_drift, float y_center_drift, int out_layout,
                                     int out_dtype) {
    ParameterFactory& f = ParameterFactory::instance();
    return rb200_crop_resize(ctx, in, dest_width, dest_height, is_output, f.create_float(area), f.create_float(aspect_ratio),
                             f.create_float(x_center_drift), f.create_float(y_center_drift), out_layout, out_dtype);
}

rb200_tensor rb200_roi_resize(rb200_context ctx, rb200_tensor in, unsigned dest_width, unsigned dest_height, int is_output,
                              unsigned roi_h, unsigned roi_w, float roi_pos_x, float roi_pos_y, int interpolation, int out_layout,
                              int out_dtype) {
    API_BEGIN
    if (dest_width == 0 || dest_height == 0) RB200_THROW("ROI Resize needs to receive non-zero destination dimensions");
    Node window;
    window.kind = NodeKind::CROP;
    window.crop.mode = CropSpec::ABSOLUTE;
    window.crop.crop_w = roi_w;
    window.crop.crop_h = roi_h;
    window.crop.x1 = (unsigned)roi_pos_x;     // the reference stores the two floats in unsigned fields
    window.crop.y1 = (unsigned)roi_pos_y;
    TensorImpl* cut = p->add_node(std::move(window), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, ROCAL_NHWC, ROCAL_UINT8, false);
    Node nd;
    nd.kind = NodeKind::RESIZE;
    nd.interpolation = resize_interpolation(interpolation);
    nd.dest_w = dest_width;
    nd.dest_h = dest_height;
    nd.scaling_mode = ROCAL_SCALING_MODE_STRETCH;
    return finish(p, std::move(nd), cut, dest_width, dest_height, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_crop_fixed(rb200_context ctx, rb200_tensor in, unsigned crop_width, unsigned crop_height, int is_output,
                              float crop_pos_x, float crop_pos_y, int out_layout, int out_dtype) {
    API_BEGIN
    if (crop_width == 0 || crop_height == 0) RB200_THROW("Crop node needs to receive non-zero destination dimensions");
    Node nd;
    nd.kind = NodeKind::CROP;
    nd.crop.mode = CropSpec::ABSOLUTE;
    nd.crop.crop_w = crop_width;
    nd.crop.crop_h = crop_height;
    nd.crop.x1 = (unsigned)crop_pos_x;
    nd.crop.y1 = (unsigned)crop_pos_y;
    return finish(p, std::move(nd), T(in), crop_width, crop_height, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_crop_center_fixed(rb200_context ctx, rb200_tensor in, unsigned crop_width, unsigned crop_height,
                                     int is_output, int out_layout, int out_dtype) {
    API_BEGIN
    if (crop_width == 0 || crop_height == 0) RB200_THROW("Crop node needs to receive non-zero destination dimensions");
    Node nd;
    nd.kind = NodeKind::CROP;
    nd.crop.mode = CropSpec::FIXED_ANCHOR;
    nd.crop.crop_w = crop_width;
    nd.crop.crop_h = crop_height;
    nd.crop.anchor_x = 0.5f;
    nd.crop.anchor_y = 0.5f;
    return finish(p, std::move(nd), T(in), crop_width, crop_height, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_resize_crop_mirror_fixed(rb200_context ctx, rb200_tensor in, unsigned dest_width, unsigned dest_height,
                                            int is_output, unsigned crop_h, unsigned crop_w, rb200_param mirror,
                                            int out_layout, int out_dtype) {
    API_BEGIN
    if (dest_width == 0 || dest_height == 0) RB200_THROW("Crop Mirror node needs tp receive non-zero destination dimensions");
    Node nd;
    nd.kind = NodeKind::RESIZE_CROP_MIRROR;
    nd.dest_w = dest_width;
    nd.dest_h = dest_height;
    nd.crop.mode = CropSpec::ABSOLUTE;
    nd.crop.crop_w = crop_w;
    nd.crop.crop_h = crop_h;
    nd.mirror = int_param(mirror, 0, 1);
    return finish(p, std::move(nd), T(in), dest_width, dest_height, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_resize_crop_mirror(rb200_context ctx, rb200_tensor in, unsigned dest_width, unsigned dest_height,
                                      int is_output, rb200_param crop_height, rb200_param crop_width, rb200_param mirror,
                                      int out_layout, int out_dtype) {
    API_BEGIN
    if (dest_width == 0 || dest_height == 0) RB200_THROW("Crop Mirror node needs tp receive non-zero destination dimensions");
    Node nd;
    nd.kind = NodeKind::RESIZE_CROP_MIRROR;
    nd.dest_w = dest_width;
    nd.dest_h = dest_height;
    nd.crop.mode = CropSpec::RANDOM;
    nd.crop.h_factor = float_param(crop_height, 0.55f, 0.95f);
    nd.crop.w_factor = float_param(crop_width, 0.55f, 0.95f);
    nd.crop.x_drift = float_param(nullptr, 0.01f, 0.99f);
    nd.crop.y_drift = float_param(nullptr, 0.01f, 0.99f);
    nd.mirror = int_param(mirror, 0, 1);
    return finish(p, std::move(nd), T(in), dest_width, dest_height, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_ssd_random_crop(rb200_context ctx, rb200_tensor in, int is_output, int num_of_attempts, int out_layout,
                                   int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::SSD_RANDOM_CROP;
    nd.ssd_attempts = num_of_attempts > 0 ? num_of_attempts : 20;
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_flip(rb200_context ctx, rb200_tensor in, int is_output, rb200_param horizontal, rb200_param vertical,
                        int out_layout, int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::FLIP;
    nd.flip_h = int_param(horizontal, 0, 1);
    nd.flip_v = int_param(vertical, 0, 1);
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

// Default ranges: include/augmentations/color_augmentations/node_*.h (ALPHA_RANGE, BETA_RANGE, ...).
rb200_tensor rb200_brightness(rb200_context ctx, rb200_tensor in, int is_output, rb200_param alpha, rb200_param beta,
                              int out_layout, int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::BRIGHTNESS;
    nd.color[0] = float_param(alpha, 0.1f, 1.95f);
    nd.color[1] = float_param(beta, 0.f, 25.f);
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_contrast(rb200_context ctx, rb200_tensor in, int is_output, rb200_param factor, rb200_param center,
                            int out_layout, int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::CONTRAST;
    nd.color[0] = float_param(factor, 0.1f, 1.95f);
    nd.color[1] = float_param(center, 60.f, 90.f);
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

// rocalExposure / rocalGamma / rocalColorTemp (rocal_api_augmentation.h:763, 269, 667; default ranges
// node_exposure.h:42, node_gamma.h:41, node_color_temperature.h:43). The reference holds no arithmetic for them
// (RPP): exposure is x * 2^factor, gamma 255 * (x/255)^gamma, colour temperature R + adjustment / B - adjustment.
rb200_tensor rb200_exposure(rb200_context ctx, rb200_tensor in, int is_output, rb200_param exposure_factor, int out_layout,
                            int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::EXPOSURE;
    nd.color[0] = float_param(exposure_factor, 0.15f, 0.95f);
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_gamma(rb200_context ctx, rb200_tensor in, int is_output, rb200_param gamma, int out_layout, int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::GAMMA;
    nd.color[0] = float_param(gamma, 0.3f, 7.00f);
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_color_temp(rb200_context ctx, rb200_tensor in, int is_output, rb200_param adjustment, int out_layout,
                              int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::COLOR_TEMP;
    nd.adjustment = int_param(adjustment, -99, 99);
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

// rocalBlend (rocal_api_augmentation.h:382; default ratio range node_blend.h:42): output = input1*ratio + input2*(1-ratio).
rb200_tensor rb200_blend(rb200_context ctx, rb200_tensor in, rb200_tensor in2, int is_output, rb200_param ratio, int out_layout,
                         int out_dtype) {
    API_BEGIN
    if (in2 == nullptr) {
        std::cerr << "[ERR] Invalid input image\n";
        return nullptr;
    }
    Node nd;
    nd.kind = NodeKind::BLEND;
    nd.color[0] = float_param(ratio, 0.1f, 0.9f);
    RocalTensorLayout lay = (RocalTensorLayout)out_layout;
    return static_cast<rocalTensor*>(p->add_node(std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, lay,
                                                 (RocalTensorOutputType)out_dtype, is_output != 0, T(in2)));
    API_END
}

// rocalNormalize (rocal_api_augmentation.h:1294, rocal_api_augmentation.cpp:2288-2308): axes of the per-sample
// tensor (0 = height, 1 = width, 2 = channel for the NHWC images of this pipeline) whose extent is reduced when a
// statistic is computed; an empty mean / std_dev list asks for that statistic to be computed (node_normalize.cpp:34-41).
rb200_tensor rb200_normalize(rb200_context ctx, rb200_tensor in, const unsigned* axes, unsigned num_axes, const float* mean,
                             unsigned num_mean, const float* std_dev, unsigned num_std, int is_output, float scale, float shift,
                             int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::NORMALIZE;
    for (unsigned k = 0; k < num_axes; k++) {
        if (!axes || axes[k] > 2) RB200_THROW("rocalNormalize: axes are 0 (height), 1 (width) or 2 (channel)");
        nd.axis_mask |= 1 << axes[k];
    }
    if (num_mean) nd.stat_mean.assign(mean, mean + num_mean);
    if (num_std) nd.stat_std.assign(std_dev, std_dev + num_std);
    if ((num_mean == 0 || num_std == 0) && nd.axis_mask == 0)
        RB200_THROW("rocalNormalize: axes must name what a computed mean / standard deviation is taken over");
    if ((num_mean && num_mean != 1 && num_mean != 3) || (num_std && num_std != 1 && num_std != 3))
        RB200_THROW("rocalNormalize: mean and std_dev hold one value or one per channel");
    nd.stat_scale = scale;
    nd.stat_shift = shift;
    if (out_dtype != ROCAL_FP32 && out_dtype != ROCAL_FP16) RB200_THROW("rocalNormalize: the output is FP32 or FP16");
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, ROCAL_NHWC, out_dtype, is_output);
    API_END
}

// rocalTranspose (rocal_api_augmentation.h:1338, rocal_api_augmentation.cpp:2349-2378): perm over the per-sample axes
// (height, width, channel); the output's maximum shape is the permuted maximum shape of the input.
rb200_tensor rb200_transpose(rb200_context ctx, rb200_tensor in, const unsigned* perm, unsigned num_perm, int is_output,
                             int out_layout) {
    API_BEGIN
    if (!perm || num_perm != 3) RB200_THROW("Transpose permutation must match with the input dims");
    Node nd;
    nd.kind = NodeKind::TRANSPOSE;
    int seen = 0;
    for (int k = 0; k < 3; k++) {
        if (perm[k] > 2) RB200_THROW("rocalTranspose: perm holds 0, 1 and 2");
        nd.perm[k] = (int)perm[k];
        seen |= 1 << perm[k];
    }
    if (seen != 7) RB200_THROW("rocalTranspose: perm is not a permutation");
    TensorImpl* tin = T(in);
    rb200_tensor out = finish(p, std::move(nd), tin, (unsigned)tin->max_w, (unsigned)tin->max_h,
                              out_layout == ROCAL_NONE ? ROCAL_NHWC : out_layout, ROCAL_UINT8, is_output);
    if (out) {
        const size_t d[3] = {(size_t)tin->max_h, (size_t)tin->max_w, 3};
        T(out)->custom_dims = {(size_t)tin->n, d[perm[0]], d[perm[1]], d[perm[2]]};
    }
    return out;
    API_END
}

rb200_tensor rb200_hue(rb200_context ctx, rb200_tensor in, int is_output, rb200_param hue, int out_layout, int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::HUE;
    nd.color[2] = float_param(hue, -359.0f, 359.0f);
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_saturation(rb200_context ctx, rb200_tensor in, int is_output, rb200_param sat, int out_layout,
                              int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::SATURATION;
    nd.color[3] = float_param(sat, -0.5f, 0.5f);
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_color_twist(rb200_context ctx, rb200_tensor in, int is_output, rb200_param alpha, rb200_param beta,
                               rb200_param hue, rb200_param sat, int out_layout, int out_dtype) {
    API_BEGIN
    Node nd;
    nd.kind = NodeKind::COLOR_TWIST;
    nd.color[0] = float_param(alpha, 0.1f, 1.95f);
    nd.color[1] = float_param(beta, 0.1f, 25.0f);
    nd.color[2] = float_param(hue, 5.0f, 170.0f);
    nd.color[3] = float_param(sat, 0.1f, 0.4f);
    return finish(p, std::move(nd), T(in), (unsigned)T(in)->max_w, (unsigned)T(in)->max_h, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_warp_affine(rb200_context ctx, rb200_tensor in, int is_output, unsigned dest_height, unsigned dest_width,
                               rb200_param x0, rb200_param x1, rb200_param y0, rb200_param y1, rb200_param o0,
                               rb200_param o1, int interpolation, int out_layout, int out_dtype) {
    API_BEGIN
    check_interpolation(interpolation);
    if (dest_width == 0 || dest_height == 0) {
        dest_width = (unsigned)T(in)->max_w;
        dest_height = (unsigned)T(in)->max_h;
    }
    Node nd;
    nd.kind = NodeKind::WARP_AFFINE;
    // COEFFICIENT_RANGE_1 for x0/y1, _0 for x1/y0, _OFFSET for o0/o1 (node_warp_affine.h:50-52, .cpp:30-35)
    nd.affine[0] = float_param(x0, 0.65f, 1.35f);
    nd.affine[1] = float_param(x1, -0.35f, 0.35f);
    nd.affine[2] = float_param(y0, -0.35f, 0.35f);
    nd.affine[3] = float_param(y1, 0.65f, 1.35f);
    nd.affine[4] = float_param(o0, -10.0f, 10.0f);
    nd.affine[5] = float_param(o1, -10.0f, 10.0f);
    return finish(p, std::move(nd), T(in), dest_width, dest_height, out_layout, out_dtype, is_output);
    API_END
}

rb200_tensor rb200_rotate(rb200_context ctx, rb200_tensor in, int is_output, rb200_param angle, unsigned dest_width,
                          unsigned dest_height, int interpolation, int out_layout, int out_dtype) {
    API_BEGIN
    check_interpolation(interpolation);
    if (dest_width == 0 || dest_height == 0) {
        dest_width = (unsigned)T(in)->max_w;
        dest_height = (unsigned)T(in)->max_h;
    }
    Node nd;
    nd.kind = NodeKind::ROTATE;
    nd.angle = float_param(angle, 0.f, 180.f);   // ROTATE_ANGLE_RANGE, node_rotate.h:47
    return finish(p, std::move(nd), T(in), dest_width, dest_height, out_layout, out_dtype, is_output);
    API_END
}

// ---- outputs ----
int rb200_set_outputs(rb200_context ctx, const rb200_tensor* tensors, size_t n) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (P(ctx)->verified()) RB200_THROW("outputs must be set before rocalVerify");
        for (size_t i = 0; i < n; i++) {
            if (!tensors || !tensors[i]) RB200_THROW("rocalSetOutputs: not a tensor of this context");
            P(ctx)->mark_output(T(tensors[i]));
        }
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}
size_t rb200_output_count(rb200_context ctx) { return ctx ? (size_t)P(ctx)->outputs()->size() : 0; }
rb200_tensor rb200_output(rb200_context ctx, size_t index) { return ctx ? P(ctx)->outputs()->at(index) : nullptr; }
void* rb200_tensor_buffer(rb200_tensor t) { return t ? T(t)->buffer() : nullptr; }
unsigned rb200_tensor_num_dims(rb200_tensor t) { return t ? T(t)->num_of_dims() : 0; }
void rb200_tensor_dims(rb200_tensor t, size_t* out) {
    if (!t) return;
    auto d = T(t)->dims();
    std::copy(d.begin(), d.end(), out);
}
void rb200_tensor_strides(rb200_tensor t, size_t* out) {
    if (!t) return;
    auto d = T(t)->strides();
    std::copy(d.begin(), d.end(), out);
}
int rb200_tensor_layout(rb200_tensor t) { return t ? (int)T(t)->layout() : -1; }
int rb200_tensor_dtype(rb200_tensor t) { return t ? (int)T(t)->data_type() : -1; }
size_t rb200_tensor_data_size(rb200_tensor t) { return t ? T(t)->data_size() : 0; }
unsigned rb200_tensor_copy_data(rb200_tensor t, void* user_buffer, int mem_type) {
    return t ? T(t)->copy_data(user_buffer, (RocalOutputMemType)mem_type) : 1;
}
void rb200_tensor_copy_roi(rb200_tensor t, void* roi_buffer) {
    if (t && roi_buffer) T(t)->copy_roi(roi_buffer);
}

void* rb200_tensor_dlpack(rb200_tensor t) {
    if (!t || !T(t)->buffer()) return nullptr;
    TensorImpl* x = T(t);
    auto* m = new DLManagedTensor();
    auto dims = x->dims();
    auto strides = x->strides();
    size_t e = x->elem_size();
    m->dl_tensor.data = x->buffer();
    m->dl_tensor.device = {2 /* kDLCUDA */, x->pipe->gpu_id()};
    m->dl_tensor.ndim = (int32_t)dims.size();
    uint8_t code = (x->dtype == ROCAL_FP32 || x->dtype == ROCAL_FP16) ? 2 /* float */
                   : (x->dtype == ROCAL_UINT8 || x->dtype == ROCAL_UINT32) ? 1 /* uint */ : 0 /* int */;
    m->dl_tensor.dtype = {code, (uint8_t)(e * 8), 1};
    m->dl_tensor.shape = new int64_t[dims.size()];
    m->dl_tensor.strides = new int64_t[dims.size()];
    for (size_t k = 0; k < dims.size(); k++) {
        m->dl_tensor.shape[k] = (int64_t)dims[k];
        m->dl_tensor.strides[k] = (int64_t)(strides[k] / e);
    }
    m->dl_tensor.byte_offset = 0;
    m->manager_ctx = nullptr;
    m->deleter = dl_deleter;
    return m;
}

int rb200_device_id(rb200_context ctx) { return ctx ? P(ctx)->gpu_id() : -1; }
void* rb200_stream(rb200_context ctx) { return ctx ? (void*)P(ctx)->stream() : nullptr; }

int rb200_to_tensor(rb200_context ctx, void* out_ptr, int layout, int dtype, const float* multiplier3, const float* offset3,
                    int reverse_channels, int output_mem_type) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!out_ptr || !multiplier3 || !offset3) RB200_THROW("null argument");
        P(ctx)->to_tensor(out_ptr, layout, dtype, multiplier3, offset3, reverse_channels != 0, output_mem_type);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

// ---- box encoder ----
int rb200_box_encoder(rb200_context ctx, const float* anchors_ltrb, size_t num_anchors, float criteria, const float* means4,
                      const float* stds4, int offset, float scale) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!means4 || !stds4) RB200_THROW("means and stds must hold 4 values");
        P(ctx)->set_box_encoder(anchors_ltrb, num_anchors, criteria, means4, stds4, offset != 0, scale);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_copy_encoded_boxes_and_labels(rb200_context ctx, float* boxes_buf, int* labels_buf) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!boxes_buf || !labels_buf) RB200_THROW("null output buffer");
        P(ctx)->copy_encoded(boxes_buf, labels_buf);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_get_encoded_boxes_and_labels(rb200_context ctx, float** boxes_dev, int** labels_dev, size_t* num_anchors) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        P(ctx)->encoded(boxes_dev, labels_dev, num_anchors);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

// ---- box IoU matcher ----
int rb200_box_iou_matcher(rb200_context ctx, const float* anchors_ltrb, size_t num_anchors, float high_threshold,
                          float low_threshold, int allow_low_quality_matches) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        P(ctx)->set_box_matcher(anchors_ltrb, num_anchors, high_threshold, low_threshold, allow_low_quality_matches != 0);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_get_matched_indices(rb200_context ctx, int** matches_dev, size_t* num_anchors) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!matches_dev || !num_anchors) RB200_THROW("null output pointer");
        P(ctx)->matches(matches_dev, num_anchors);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

int rb200_copy_matched_indices(rb200_context ctx, int* matches_buf) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!matches_buf) RB200_THROW("null output buffer");
        int* dev;
        size_t a;
        P(ctx)->matches(&dev, &a);
        P(ctx)->sync_copy(matches_buf, dev, (size_t)P(ctx)->batch() * a * sizeof(int), cudaMemcpyDeviceToHost);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

size_t rb200_get_bounding_boxes(rb200_context ctx, float* ltrb, int* labels, int* counts) {
    CTX_OR(0);
    try {
        std::vector<float> b;
        std::vector<int> l, c;
        P(ctx)->current_boxes(b, l, c);
        if (ltrb) std::memcpy(ltrb, b.data(), b.size() * sizeof(float));
        if (labels) std::memcpy(labels, l.data(), l.size() * sizeof(int));
        if (counts) std::memcpy(counts, c.data(), c.size() * sizeof(int));
        return l.size();
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return 0;
    }
}

int rb200_get_crop_windows(rb200_context ctx, rb200_tensor t, unsigned* xywh) {
    CTX_OR(ROCAL_CONTEXT_INVALID);
    try {
        if (!t || !xywh) RB200_THROW("null argument");
        P(ctx)->crop_windows(T(t), xywh);
    } catch (const std::exception& e) {
        report(P(ctx), e);
        return ROCAL_RUNTIME_ERROR;
    }
    return ROCAL_OK;
}

size_t rb200_get_int_array(rb200_param p, int* out, size_t n) {
    if (!p || !out || !ParameterFactory::instance().owns(p)) return 0;
    const auto& a = IP(p)->core->array();
    size_t k = std::min(n, a.size());
    std::copy(a.begin(), a.begin() + k, out);
    return k;
}

size_t rb200_get_batch_int_array(rb200_context ctx, rb200_param p, int* out, size_t n) {
    if (!ctx || !p || !out || !ParameterFactory::instance().owns(p)) return 0;
    return P(ctx)->batch_int_array(IP(p)->core, out, n);
}

size_t rb200_get_batch_float_array(rb200_context ctx, rb200_param p, float* out, size_t n) {
    if (!ctx || !p || !out || !ParameterFactory::instance().owns(p)) return 0;
    return P(ctx)->batch_float_array(FP(p)->core, out, n);
}

size_t rb200_get_float_array(rb200_param p, float* out, size_t n) {
    if (!p || !out || !ParameterFactory::instance().owns(p)) return 0;
    const auto& a = FP(p)->core->array();
    size_t k = std::min(n, a.size());
    std::copy(a.begin(), a.begin() + k, out);
    return k;
}

}  // extern "C"
