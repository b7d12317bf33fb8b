#include "pipeline.h"

#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <cstdio>

#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <optional>

namespace rb200 {

static void read_file(const std::string& path, std::vector<unsigned char>& out) {
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open " + path);
    std::fseek(f, 0, SEEK_END);
    long len = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    if (len <= 0) {
        std::fclose(f);
        throw std::runtime_error("empty file " + path);
    }
    out.resize((size_t)len);
    size_t got = std::fread(out.data(), 1, (size_t)len, f);
    std::fclose(f);
    if (got != (size_t)len) throw std::runtime_error("short read on " + path);
}

static inline unsigned long long now_us() {
    return (unsigned long long)std::chrono::duration_cast<std::chrono::microseconds>(
               std::chrono::steady_clock::now().time_since_epoch())
        .count();
}

int log_level() {
    static const int level = [] {
        const char* e = std::getenv("RB200_LOG_LEVEL");
        return e && *e ? std::atoi(e) : 1;
    }();
    return level;
}

// A named range on the profiler's timeline (NVTX; costs a few nanoseconds when no tool is attached).
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};

// ------------------------------------------------------------------------------------------
// Host-side size rules
// ------------------------------------------------------------------------------------------

// Target size of one resized sample: ResizeNode::adjust_out_roi_size
// (source/augmentations/geometry_augmentations/node_resize.cpp:98-138).
static void resize_target(unsigned src_w, unsigned src_h, unsigned dst_w, unsigned dst_h, int mode, unsigned max_w,
                          unsigned max_h, unsigned& out_w, unsigned& out_h) {
    bool has_max = (max_w | max_h) > 0;
    if (mode == ROCAL_SCALING_MODE_MIN_MAX) {
        // ResizeMirrorNormalizeNode::adjust_out_roi_size (node_resize_mirror_normalize.cpp:138-160): max_w holds the
        // minimum size, max_h the maximum size.
        unsigned min_size = max_w, max_size = max_h, size = min_size;
        float min_o = static_cast<float>(std::min(src_w, src_h)), max_o = static_cast<float>(std::max(src_w, src_h));
        if (max_o / min_o * size > max_size) size = static_cast<size_t>(std::round(max_size * min_o / max_o));
        if (src_w < src_h) {
            dst_w = size;
            dst_h = static_cast<size_t>(size * src_h / src_w);
        } else {
            dst_h = size;
            dst_w = static_cast<size_t>(size * src_w / src_h);
        }
    } else if (mode == ROCAL_SCALING_MODE_STRETCH) {
        if (!dst_w) dst_w = src_w;
        if (!dst_h) dst_h = src_h;
        if (has_max) {
            if (max_w) dst_w = std::min(dst_w, max_w);
            if (max_h) dst_h = std::min(dst_h, max_h);
        }
    } else if (mode == ROCAL_SCALING_MODE_DEFAULT) {
        if ((!dst_w) & (dst_h != 0)) {
            dst_w = (unsigned)std::lround(src_w * (static_cast<float>(dst_h) / src_h));
        } else if ((!dst_h) & (dst_w != 0)) {
            dst_h = (unsigned)std::lround(src_h * (static_cast<float>(dst_w) / src_w));
        }
        if (has_max) {
            if (max_w) dst_w = std::min(dst_w, max_w);
            if (max_h) dst_h = std::min(dst_h, max_h);
        }
    } else {
        float scale = 1.0f;
        float scale_w = static_cast<float>(dst_w) / src_w;
        float scale_h = static_cast<float>(dst_h) / src_h;
        if (mode == ROCAL_SCALING_MODE_NOT_SMALLER) {
            scale = std::max(scale_w, scale_h);
        } else if (mode == ROCAL_SCALING_MODE_NOT_LARGER) {
            scale = (scale_w > 0 && scale_h > 0) ? std::min(scale_w, scale_h) : ((scale_w > 0) ? scale_w : scale_h);
        }
        if (has_max) {
            if (max_w) scale = std::min(scale, static_cast<float>(max_w) / src_w);
            if (max_h) scale = std::min(scale, static_cast<float>(max_h) / src_h);
        }
        if ((scale_h != scale) || (!dst_h)) dst_h = (unsigned)std::lround(src_h * scale);
        if ((scale_w != scale) || (!dst_w)) dst_w = (unsigned)std::lround(src_w * scale);
    }
    out_w = dst_w;
    out_h = dst_h;
}

void CropSpec::update(const std::vector<int>& in_w, const std::vector<int>& in_h) {
    size_t n = in_w.size();
    x1v.resize(n);
    y1v.resize(n);
    cwv.resize(n);
    chv.resize(n);
    for (size_t i = 0; i < n; i++) {
        unsigned w = (unsigned)in_w[i], h = (unsigned)in_h[i];
        if (mode == RANDOM_AREA) {
            // up to five (area, aspect) draws for a window strictly smaller than the image, placed by the two
            // drifts (the vertical one is renewed twice per success); otherwise the central crop clamped to
            // the aspect range 0.75 .. 1.333
            const float kAspectLo = 0.7500f, kAspectHi = 1.333f;
            bool placed = false;
            unsigned cw = 0, ch = 0;
            for (int attempt = 0; attempt < 5 && !placed; attempt++) {
                area->renew();
                aspect->renew();
                const float a = area->get(), r = aspect->get();
                const double target = (double)(a * (float)h * (float)w);
                cw = static_cast<unsigned>(static_cast<size_t>(std::sqrt(target * (double)r)));
                ch = static_cast<unsigned>(static_cast<size_t>(std::sqrt(target * (double)(1 / r))));
                if (ch < h && cw < w) {
                    x_drift->renew();
                    y_drift->renew();
                    y_drift->renew();
                    const float xd = x_drift->get(), yd = y_drift->get();
                    x1v[i] = static_cast<unsigned>(static_cast<size_t>(xd * (float)(w - cw)));
                    y1v[i] = static_cast<unsigned>(static_cast<size_t>(yd * (float)(h - ch)));
                    placed = true;
                }
            }
            if (!placed) {
                const float in_ratio = (float)w / (float)h;
                if (in_ratio < kAspectLo) {
                    cw = w;
                    ch = static_cast<unsigned>((float)cw / kAspectLo);
                } else if (in_ratio > kAspectHi) {
                    ch = h;
                    cw = static_cast<unsigned>((float)ch * kAspectHi);
                } else {
                    ch = h;
                    cw = w;
                }
                x1v[i] = (w - cw) / 2;
                y1v[i] = (h - ch) / 2;
            }
            cwv[i] = cw;
            chv[i] = ch;
        } else if (mode != RANDOM) {
            cwv[i] = (crop_w <= w && crop_w > 0) ? crop_w : w;
            chv[i] = (crop_h <= h && crop_h > 0) ? crop_h : h;
            if (mode == FIXED_ANCHOR) {
                float ax = next_anchor_x.size() == n ? next_anchor_x[i] : anchor_x;
                float ay = next_anchor_y.size() == n ? next_anchor_y[i] : anchor_y;
                x1v[i] = static_cast<unsigned>(static_cast<size_t>(std::nearbyintf(ax * (w - cwv[i]))));
                y1v[i] = static_cast<unsigned>(static_cast<size_t>(std::nearbyintf(ay * (h - chv[i]))));
            } else {
                x1v[i] = (x1 >= w) ? 0 : x1;
                y1v[i] = (y1 >= h) ? 0 : y1;
            }
        } else {
            h_factor->renew();
            float hf = h_factor->get();
            w_factor->renew();
            float wf = w_factor->get();
            cwv[i] = static_cast<unsigned>(static_cast<size_t>(wf * w));
            chv[i] = static_cast<unsigned>(static_cast<size_t>(hf * h));
            x_drift->renew();
            y_drift->renew();
            float xd = x_drift->get(), yd = y_drift->get();
            x1v[i] = static_cast<unsigned>(static_cast<size_t>(xd * (w - cwv[i])));
            y1v[i] = static_cast<unsigned>(static_cast<size_t>(yd * (h - chv[i])));
        }
        // The window handed to the kernel never leaves the image (the reference clamps x2/y2 only).
        if (x1v[i] >= w) x1v[i] = w ? w - 1 : 0;
        if (y1v[i] >= h) y1v[i] = h ? h - 1 : 0;
        cwv[i] = std::max(1u, std::min(cwv[i], w - x1v[i]));
        chv[i] = std::max(1u, std::min(chv[i], h - y1v[i]));
    }
    next_anchor_x.clear();
    next_anchor_y.clear();
}

// ------------------------------------------------------------------------------------------
// Tensors
// ------------------------------------------------------------------------------------------

TensorImpl::TensorImpl(Pipeline* p, int id_, int n_, int mw, int mh, RocalTensorOutputType dt, RocalTensorLayout l,
                       bool out, bool src)
    : pipe(p), id(id_), n(n_), max_w(mw), max_h(mh), dtype(dt), lay(l), is_output(out), is_source(src) {
    roi_w.assign(n, mw);
    roi_h.assign(n, mh);
    user_roi.assign((size_t)n * 4, 0);
}

std::vector<size_t> TensorImpl::dims() {
    if (!custom_dims.empty()) return custom_dims;
    if (lay == ROCAL_NCHW) return {(size_t)n, 3, (size_t)max_h, (size_t)max_w};
    return {(size_t)n, (size_t)max_h, (size_t)max_w, 3};
}

std::vector<size_t> TensorImpl::strides() {
    size_t e = elem_size();
    if (!custom_dims.empty()) {
        std::vector<size_t> st(custom_dims.size(), e);
        for (int k = (int)custom_dims.size() - 2; k >= 0; k--) st[k] = st[k + 1] * custom_dims[k + 1];
        return st;
    }
    if (lay == ROCAL_NCHW) return {(size_t)3 * max_h * max_w * e, (size_t)max_h * max_w * e, (size_t)max_w * e, e};
    return {(size_t)max_h * max_w * 3 * e, (size_t)max_w * 3 * e, 3 * e, e};
}

unsigned TensorImpl::copy_data(void* user_buffer, RocalOutputMemType external_mem_type) {
    if (!user_buffer) return 1;
    if (host_mem) {
        if (data_size() == 0) return 0;
        if (!current) return 1;
        try {
            if (external_mem_type == ROCAL_MEMCPY_GPU)
                pipe->sync_copy(user_buffer, current, data_size(), cudaMemcpyHostToDevice);
            else
                std::memcpy(user_buffer, current, data_size());
        } catch (const std::exception& e) {
            pipe->capture_error(e.what());
            return 1;
        }
        return 0;
    }
    if (!current) return 1;
    try {
        pipe->sync_copy(user_buffer, current, data_size(),
                        external_mem_type == ROCAL_MEMCPY_GPU ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost);
    } catch (const std::exception& e) {
        pipe->capture_error(e.what());
        return 1;
    }
    return 0;
}

unsigned TensorImpl::copy_data(void* user_buffer, unsigned x_offset, unsigned y_offset, unsigned max_cols, unsigned max_rows) {
    // Copies the window (x_offset, y_offset, max_cols, max_rows) of every sample to host memory, tightly packed.
    if (!current || !user_buffer) return 1;
    if (x_offset + max_cols > (unsigned)max_w || y_offset + max_rows > (unsigned)max_h) return 1;
    size_t e = elem_size();
    try {
        cudaSetDevice(pipe->gpu_id());
        uint8_t* dst = (uint8_t*)user_buffer;
        const uint8_t* src = (const uint8_t*)current;
        if (lay == ROCAL_NCHW) {
            for (int i = 0; i < n * 3; i++) {
                RB200_CUDA(cudaMemcpy2D(dst + (size_t)i * max_rows * max_cols * e, max_cols * e,
                                        src + ((size_t)i * max_h * max_w + (size_t)y_offset * max_w + x_offset) * e,
                                        (size_t)max_w * e, max_cols * e, max_rows, cudaMemcpyDeviceToHost));
            }
        } else {
            for (int i = 0; i < n; i++) {
                RB200_CUDA(cudaMemcpy2D(dst + (size_t)i * max_rows * max_cols * 3 * e, max_cols * 3 * e,
                                        src + ((size_t)i * max_h * max_w + (size_t)y_offset * max_w + x_offset) * 3 * e,
                                        (size_t)max_w * 3 * e, max_cols * 3 * e, max_rows, cudaMemcpyDeviceToHost));
            }
        }
    } catch (const std::exception& ex) {
        pipe->capture_error(ex.what());
        return 1;
    }
    return 0;
}

void TensorImpl::copy_roi(void* roi_buffer) { std::memcpy(roi_buffer, user_roi.data(), user_roi.size() * sizeof(unsigned)); }

// ------------------------------------------------------------------------------------------
// Pipeline: construction and graph building
// ------------------------------------------------------------------------------------------

Pipeline::Pipeline(size_t batch, int gpu_id, size_t depth, RocalTensorOutputType out_dtype)
    : _batch(batch), _gpu_id(gpu_id), _depth(depth < 2 ? 2 : depth), _out_dtype(out_dtype) {
    if (batch == 0 || batch > 65535) RB200_THROW("batch size must be in [1, 65535]");
    int count = 0;
    RB200_CUDA(cudaGetDeviceCount(&count));
    if (gpu_id < 0 || gpu_id >= count) RB200_THROW("invalid gpu_id " + std::to_string(gpu_id));
    RB200_CUDA(cudaSetDevice(gpu_id));
    RB200_CUDA(cudaStreamCreateWithFlags(&_stream, cudaStreamNonBlocking));
    RB200_CUDA(cudaStreamCreateWithFlags(&_meta_stream, cudaStreamNonBlocking));
    RB200_CUDA(cudaEventCreateWithFlags(&_meta_done, cudaEventDisableTiming));
    RB200_CUDA(cudaEventCreateWithFlags(&_box_stage_free, cudaEventDisableTiming));
}

Pipeline::~Pipeline() {
    {
        std::lock_guard<std::mutex> lk(_m);
        _stop = true;
    }
    _cv_work.notify_all();
    _cv_ready.notify_all();
    if (_worker.joinable()) _worker.join();
    if (log_level() >= 2) {
        std::fprintf(stderr, "[rb200] host time (us): load %llu, decode %llu, tables+launch %llu, transfer %llu\n", _t_load.load(),
                     _t_decode.load(), _t_process.load(), _t_transfer.load());
        for (const StepTiming& t : _step_timing)
            if (t.batches)
                std::fprintf(stderr, "[rb200]   %-12s %10.1f us device time per batch over %llu batches\n", t.name.c_str(),
                             t.gpu_us / (double)t.batches, t.batches);
    }
    cudaSetDevice(_gpu_id);
    if (_stream) cudaStreamSynchronize(_stream);
    if (_meta_stream) cudaStreamSynchronize(_meta_stream);
    for (auto& t : _tensors) {
        for (void* p : t->ring) cudaFree(p);
        if (t->scratch) cudaFree(t->scratch);
    }
    for (auto& s : _slots) {
        for (cudaEvent_t ev : s.step_ev)
            if (ev) cudaEventDestroy(ev);
        if (s.done) cudaEventDestroy(s.done);
        if (s.consumer_done) cudaEventDestroy(s.consumer_done);
        if (s.h_status) cudaFreeHost(s.h_status);
        if (s.d_tables) cudaFree(s.d_tables);
        if (s.h_tables) cudaFreeHost(s.h_tables);
        if (s.d_enc_boxes) cudaFree(s.d_enc_boxes);
        if (s.d_enc_labels) cudaFree(s.d_enc_labels);
        if (s.d_matches) cudaFree(s.d_matches);
    }
    for (int k = 0; k < 2; k++) {
        if (_arena[k]) cudaFree(_arena[k]);
        if (_arena_free[k]) cudaEventDestroy(_arena_free[k]);
    }
    if (_d_anchors) cudaFree(_d_anchors);
    if (_d_match_anchors) cudaFree(_d_match_anchors);
    if (_norm_scratch) cudaFree(_norm_scratch);
    if (_d_boxes) cudaFree(_d_boxes);
    if (_d_labels) cudaFree(_d_labels);
    if (_d_offsets) cudaFree(_d_offsets);
    if (_h_box_stage) cudaFreeHost(_h_box_stage);
    if (_meta_done) cudaEventDestroy(_meta_done);
    if (_box_stage_free) cudaEventDestroy(_box_stage_free);
    if (_meta_stream) cudaStreamDestroy(_meta_stream);
    if (_stream) cudaStreamDestroy(_stream);
}

bool Pipeline::owns(const void* t) const {
    for (auto& p : _tensors)
        if (p.get() == t) return true;
    return false;
}

TensorImpl* Pipeline::add_source(unsigned max_w, unsigned max_h, bool is_output) {
    if (_verified) RB200_THROW("the graph is already verified");
    if (_source >= 0) RB200_THROW("only one external source per context is supported");
    if (max_w == 0 || max_h == 0) RB200_THROW("max_width and max_height must be given for raw uncompressed input");
    int id = (int)_tensors.size();
    _tensors.emplace_back(new TensorImpl(this, id, (int)_batch, (int)max_w, (int)max_h, ROCAL_UINT8, ROCAL_NHWC, is_output, true));
    _source = id;
    return _tensors.back().get();
}

// rocalJpegFileSourceSingleShard (rocal_api_data_loaders.h:80-90): the source tensor plus a folder reader that
// feeds the pipeline by itself.
TensorImpl* Pipeline::add_file_source(const std::string& root, unsigned shard_id, unsigned shard_count, bool shuffle, bool loop,
                                      unsigned max_w, unsigned max_h, bool is_output, int last_batch_policy,
                                      bool pad_last_batch_repeated) {
    if (max_w == 0 || max_h == 0) RB200_THROW("max_width and max_height must be given (ROCAL_USE_USER_GIVEN_SIZE): they bound the decoded size");
    std::unique_ptr<FileSource> fs;
    if (_file_list.empty())
        fs.reset(new FileSource(root, _batch, shard_id, shard_count, shuffle, loop, last_batch_policy, pad_last_batch_repeated,
                                ParameterFactory::instance().get_seed()));
    else
        fs.reset(new FileSource(read_file_list(_file_list, root), false, _batch, shard_id, shard_count, shuffle, loop,
                                last_batch_policy, pad_last_batch_repeated, ParameterFactory::instance().get_seed()));
    TensorImpl* t = add_source(max_w, max_h, is_output);
    _files = std::move(fs);
    return t;
}

// rocalJpegCOCOFileSourceSingleShard + rocalCreateCOCOReader (rocal_api_data_loaders.h:257-269,
// rocal_api_meta_data.h:89): the images named by the annotation file, found under `root`, with their boxes.
TensorImpl* Pipeline::add_coco_source(const std::string& root, const std::string& json_path, bool avoid_class_remapping,
                                      unsigned shard_id, unsigned shard_count, bool shuffle, bool loop, unsigned max_w, unsigned max_h,
                                      bool is_output, int last_batch_policy, bool pad_last_batch_repeated) {
    if (max_w == 0 || max_h == 0) RB200_THROW("max_width and max_height must be given (ROCAL_USE_USER_GIVEN_SIZE): they bound the decoded size");
    std::vector<CocoImage> images = read_coco_annotations(json_path, avoid_class_remapping);
    std::vector<FileEntry> entries;
    for (CocoImage& im : images) {
        FileEntry e;
        e.path = root + "/" + im.file_name;
        FILE* f = std::fopen(e.path.c_str(), "rb");     // images of the file that are not on disk are left out
        if (!f) continue;
        std::fclose(f);
        e.name = im.file_name;
        e.label = (int)im.id;            // a detection sample has no class label: the slot carries the image id
        e.boxes = std::move(im.boxes);
        e.box_labels = std::move(im.labels);
        entries.push_back(std::move(e));
    }
    if (entries.empty()) RB200_THROW("none of the images named in " + json_path + " was found under " + root);
    std::unique_ptr<FileSource> fs(new FileSource(std::move(entries), true, _batch, shard_id, shard_count, shuffle, loop, last_batch_policy,
                                                  pad_last_batch_repeated, ParameterFactory::instance().get_seed()));
    TensorImpl* t = add_source(max_w, max_h, is_output);
    _files = std::move(fs);
    _coco_source = true;
    return t;
}

// Keeps the ring busy from the folder reader: one batch per free slot.
void Pipeline::top_up() {
    if (!_files) return;
    for (;;) {
        {
            std::lock_guard<std::mutex> lk(_m);
            if (_in_flight >= _depth) return;
        }
        FileBatch fb;
        if (!_files->next(fb)) return;
        InputBatch b;
        b.kind = InputBatch::ENCODED;
        b.n = _batch;
        b.paths = std::move(fb.paths);
        b.names = std::move(fb.names);
        b.file_labels = std::move(fb.labels);
        b.padded = fb.padded;
        if (fb.has_boxes) {
            // an image without annotations keeps one empty box with label 0, as the reference's metadata graph
            // does (bounding_box_graph.cpp:53-55)
            std::vector<float> bx;
            std::vector<int> bl, bc;
            size_t at = 0;
            for (size_t i = 0; i < fb.counts.size(); i++) {
                const int c = fb.counts[i];
                if (c == 0) {
                    bx.insert(bx.end(), {0.f, 0.f, 0.f, 0.f});
                    bl.push_back(0);
                    bc.push_back(1);
                } else {
                    bx.insert(bx.end(), fb.boxes.begin() + at * 4, fb.boxes.begin() + (at + c) * 4);
                    bl.insert(bl.end(), fb.box_labels.begin() + at, fb.box_labels.begin() + at + c);
                    bc.push_back(c);
                }
                at += (size_t)c;
            }
            stage_boxes(bx.data(), bl.data(), bc.data(), bc.size());
        }
        feed(std::move(b));
    }
}

void Pipeline::set_random_bbox_crop(bool all_boxes_overlap, bool has_shape, uint32_t seed) {
    if (_verified) RB200_THROW("rocalRandomBBoxCrop must be called before rocalVerify");
    _bbox_crop = std::make_unique<BBoxCropSampler>(seed, all_boxes_overlap, has_shape);
}

void Pipeline::bbox_crop_windows(float* xywh) {
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    const Slot& s = _slots[_held];
    if (s.bbox_crop_windows.size() != _batch * 4) RB200_THROW("the current batch was not cut by rocalRandomBBoxCrop");
    if (xywh) std::memcpy(xywh, s.bbox_crop_windows.data(), s.bbox_crop_windows.size() * sizeof(float));
}

void Pipeline::set_random_crop_decoder(const RandomCropRanges& r) {
    if (_verified) RB200_THROW("the graph is already verified");
    if (_source < 0) RB200_THROW("the context has no source yet");
    if (_tensors[_source]->is_output) RB200_THROW("the fused JPEG crop source cannot be a graph output");
    if (!(r.area_lo > 0.f) || r.area_hi < r.area_lo || !(r.aspect_lo > 0.f) || r.aspect_hi < r.aspect_lo || r.num_attempts < 1)
        RB200_THROW("fused JPEG crop: area_factor and aspect_ratio must be positive ascending pairs, num_attempts >= 1");
    _crop_dec.reset(new RandomCropWindowSampler(r, ParameterFactory::instance().get_seed()));
}

void Pipeline::decoder_crop_windows(unsigned* xywh, unsigned* batch_seed) {
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    const Slot& s = _slots[_held];
    if (s.decoder_windows.size() != _batch * 4) RB200_THROW("the current batch did not come from a fused JPEG crop source");
    if (xywh) std::memcpy(xywh, s.decoder_windows.data(), s.decoder_windows.size() * sizeof(unsigned));
    if (batch_seed) *batch_seed = s.decoder_batch_seed;
}

void Pipeline::reset_loaders() {
    if (!_files) RB200_THROW("rocalResetLoaders: the context has no file source");
    _files->reset();
    top_up();
}

void Pipeline::image_labels(int* buf) {
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    const Slot& s = _slots[_held];
    if (s.file_labels.size() != _batch) RB200_THROW("the current batch carries no labels (no file source / label reader)");
    std::memcpy(buf, s.file_labels.data(), _batch * sizeof(int));
}

// rocalGetImageLabels (rocal_api_meta_data.cpp:197-203): the labels of the current batch as a tensor list, one
// one-element int32 host tensor per sample whose buffers lie one after the other, so that at(0)->buffer() reads
// as int[batch] (what the reference's Python binding does, rocal_pybind.cpp:862-871).
TensorListImpl* Pipeline::image_label_list() {
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    const Slot& s = _slots[_held];
    if (s.file_labels.size() != _batch) RB200_THROW("the current batch carries no labels (no file source / label reader)");
    _label_values = s.file_labels;
    if (_label_t.size() != _batch) {
        _label_t.clear();
        _label_list.items.clear();
        for (size_t i = 0; i < _batch; i++) {
            std::unique_ptr<TensorImpl> l(new TensorImpl(this, -12, 1, 1, 1, ROCAL_INT32, ROCAL_NHWC, false, false));
            l->custom_dims = {1};
            l->host_mem = true;
            _label_list.items.push_back(l.get());
            _label_t.push_back(std::move(l));
        }
    }
    for (size_t i = 0; i < _batch; i++) _label_t[i]->current = &_label_values[i];
    return &_label_list;
}

// rocalGetImageId (rocal_api_meta_data.cpp:185-195): the "id" of every image of the batch in the COCO annotation file.
void Pipeline::image_ids(int* buf) {
    if (!_coco_source) RB200_THROW("rocalGetImageId needs a COCO source");
    image_labels(buf);
}

const std::vector<std::string>& Pipeline::image_names() {
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    return _slots[_held].names;
}

// rocalGetImageSizes: the size of every source image as it was read (a fused JPEG crop does not change it).
void Pipeline::source_sizes(int* wh) {
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    const auto& r = _slots[_held].source_wh;
    if (r.size() != _batch * 2) RB200_THROW("the current batch carries no image sizes");
    std::memcpy(wh, r.data(), r.size() * sizeof(int));
}

// rocalGetROIImageSizes: the valid extent of every sample after ResizeMirrorNormalize, the node that maintains this
// field in the reference (meta_node_resize_mirror_normalize.cpp:79-82); without such a node, of the first output.
void Pipeline::roi_image_sizes(int* wh) {
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    int tensor = -1;
    for (const Node& nd : _nodes)
        if (nd.kind == NodeKind::RESIZE_MIRROR_NORMALIZE) tensor = nd.out;
    if (tensor < 0) {
        if (_output_list.items.empty()) RB200_THROW("the graph has no output");
        tensor = static_cast<TensorImpl*>(_output_list.items[0])->id;
    }
    const auto& r = _slots[_held].rois[tensor];
    for (size_t i = 0; i < _batch; i++) {
        wh[i * 2] = (int)r[i * 4 + 2];
        wh[i * 2 + 1] = (int)r[i * 4 + 3];
    }
}

size_t Pipeline::last_batch_padded_size() {
    if (_held < 0) return 0;
    return _slots[_held].padded;
}

TensorImpl* Pipeline::add_node(Node node, TensorImpl* in, unsigned out_w, unsigned out_h, RocalTensorLayout lay,
                               RocalTensorOutputType dt, bool is_output, TensorImpl* in2) {
    if (_verified) RB200_THROW("the graph is already verified");
    if (!owns(in) || (in2 && !owns(in2))) RB200_THROW("input tensor does not belong to this context");
    if (in2) {
        if (in2->max_w != in->max_w || in2->max_h != in->max_h) RB200_THROW("the two inputs must have the same maximum size");
        if (in2->dtype != ROCAL_UINT8 || in2->lay != ROCAL_NHWC) RB200_THROW("the input of an augmentation must be a uint8 NHWC tensor");
        node.in2 = in2->id;
        in2->consumers++;
    }
    if (out_w == 0 || out_h == 0) RB200_THROW("output dimensions must be non-zero");
    if (lay == ROCAL_NONE) lay = in->lay;
    if (lay != ROCAL_NHWC && lay != ROCAL_NCHW) RB200_THROW("only NHWC and NCHW image layouts are supported");
    if (dt != ROCAL_UINT8 && dt != ROCAL_FP32 && dt != ROCAL_FP16) RB200_THROW("output type must be UINT8, FP32 or FP16");
    int id = (int)_tensors.size();
    _tensors.emplace_back(new TensorImpl(this, id, (int)_batch, (int)out_w, (int)out_h, dt, lay, is_output, false));
    if (is_output) _output_order.push_back(id);
    node.in = in->id;
    node.out = id;
    _tensors.back()->producer = (int)_nodes.size();
    in->consumers++;
    _nodes.push_back(std::move(node));
    return _tensors.back().get();
}

void Pipeline::set_box_encoder(const float* anchors, size_t num_anchors, float criteria, const float* means,
                               const float* stds, bool offset, float scale) {
    if (_verified) RB200_THROW("the graph is already verified");
    if (!anchors || num_anchors == 0) RB200_THROW("box encoder needs a non-empty anchor list");
    _anchors.assign(anchors, anchors + num_anchors * 4);
    _enc.num_anchors = (int32_t)num_anchors;
    _enc.criteria = criteria;
    for (int k = 0; k < 4; k++) {
        _enc.means[k] = means[k];
        _enc.inv_stds[k] = (float)(1. / stds[k]);
    }
    _enc.offset = offset ? 1 : 0;
    _enc.scale = scale;
    _box_encoder = true;
}

// rocalBoxIouMatcher (source/api/rocal_api_meta_data.cpp:474-483): matched box index per anchor.
void Pipeline::set_box_matcher(const float* anchors, size_t num_anchors, float high, float low, bool allow_low_quality) {
    if (_verified) RB200_THROW("the graph is already verified");
    if (!anchors || num_anchors == 0) RB200_THROW("box IoU matcher needs a non-empty anchor list");
    _match_anchors.assign(anchors, anchors + num_anchors * 4);
    _match.num_anchors = (int32_t)num_anchors;
    _match.high_threshold = high;
    _match.low_threshold = low;
    _match.allow_low_quality_matches = allow_low_quality ? 1 : 0;
    _box_matcher = true;
}

// ------------------------------------------------------------------------------------------
// verify(): fusion plan + allocation + worker start
// ------------------------------------------------------------------------------------------

static bool is_color(NodeKind k) {
    return k == NodeKind::BRIGHTNESS || k == NodeKind::CONTRAST || k == NodeKind::HUE || k == NodeKind::SATURATION ||
           k == NodeKind::COLOR_TWIST || k == NodeKind::EXPOSURE || k == NodeKind::GAMMA || k == NodeKind::COLOR_TEMP;
}

void Pipeline::plan() {
    auto fusable_mid = [&](int tensor_id) {
        TensorImpl* t = _tensors[tensor_id].get();
        return !t->is_output && t->consumers == 1 && t->dtype == ROCAL_UINT8 && t->lay == ROCAL_NHWC;
    };
    auto consumer_of = [&](int tensor_id) {
        for (size_t k = 0; k < _nodes.size(); k++)
            if (_nodes[k].in == tensor_id) return (int)k;
        return -1;
    };
    for (size_t k = 0; k < _nodes.size(); k++) {
        Node& nd = _nodes[k];
        if (!fusable_mid(nd.out)) continue;
        int c = consumer_of(nd.out);
        if (c < 0) continue;
        NodeKind ck = _nodes[c].kind;
        if ((nd.kind == NodeKind::CROP || nd.kind == NodeKind::SSD_RANDOM_CROP) &&
            (ck == NodeKind::RESIZE || ck == NodeKind::RESIZE_MIRROR_NORMALIZE))
            nd.absorbed_by = c;
        else if (nd.kind == NodeKind::RESIZE && ck == NodeKind::CROP_MIRROR_NORMALIZE)
            nd.absorbed_by = c;
        else if (is_color(nd.kind) && ck == NodeKind::FLIP)
            nd.absorbed_by = c;
    }
    for (size_t k = 0; k < _nodes.size(); k++) {
        Node& nd = _nodes[k];
        if (nd.absorbed_by >= 0) continue;
        Step st;
        st.out_tensor = nd.out;
        st.in_tensor = nd.in;
        auto producer_absorbed = [&](int tensor_id) {
            int p = _tensors[tensor_id]->producer;
            return (p >= 0 && _nodes[p].absorbed_by == (int)k) ? p : -1;
        };
        switch (nd.kind) {
            case NodeKind::CROP_MIRROR_NORMALIZE: {
                int r = producer_absorbed(nd.in);
                if (r >= 0) {
                    st.kind = Step::RESAMPLE;
                    st.post = (int)k;
                    st.resize = r;
                    st.in_tensor = _nodes[r].in;
                    int p = _tensors[_nodes[r].in]->producer;
                    if (p >= 0 && _nodes[p].absorbed_by == r) {
                        st.pre_crop = p;
                        st.in_tensor = _nodes[p].in;
                    }
                } else {
                    st.kind = Step::POINTWISE;
                    st.window = (int)k;
                }
                break;
            }
            case NodeKind::RESIZE:
            case NodeKind::RESIZE_MIRROR_NORMALIZE:
            case NodeKind::RESIZE_CROP_MIRROR: {
                st.kind = Step::RESAMPLE;
                st.resize = (int)k;
                int p = producer_absorbed(nd.in);
                if (p >= 0) {
                    st.pre_crop = p;
                    st.in_tensor = _nodes[p].in;
                }
                break;
            }
            case NodeKind::CROP:
            case NodeKind::SSD_RANDOM_CROP:
                st.kind = Step::POINTWISE;
                st.window = (int)k;
                break;
            case NodeKind::FLIP: {
                st.kind = Step::POINTWISE;
                st.flip = (int)k;
                int c = producer_absorbed(nd.in);
                if (c >= 0) {
                    st.color = c;
                    st.in_tensor = _nodes[c].in;
                }
                break;
            }
            case NodeKind::WARP_AFFINE:
            case NodeKind::ROTATE:
                st.kind = Step::WARP;
                st.warp = (int)k;
                break;
            case NodeKind::NORMALIZE:
                st.kind = Step::NORMALIZE;
                st.node = (int)k;
                break;
            case NodeKind::TRANSPOSE:
                st.kind = Step::TRANSPOSE;
                st.node = (int)k;
                break;
            default:
                st.kind = Step::POINTWISE;
                st.color = (int)k;
                st.in2_tensor = nd.in2;
        }
        TensorImpl* in = _tensors[st.in_tensor].get();
        TensorImpl* out = _tensors[st.out_tensor].get();
        if (in->dtype != ROCAL_UINT8 || in->lay != ROCAL_NHWC)
            RB200_THROW("the input of an augmentation must be a uint8 NHWC tensor");
        if (st.kind == Step::WARP && (out->dtype != ROCAL_UINT8 || out->lay != ROCAL_NHWC))
            RB200_THROW("WarpAffine/Rotate produce uint8 NHWC output");
        out->materialized = true;
        _steps.push_back(st);
    }
}

void Pipeline::mark_output(TensorImpl* t) {
    if (_verified) RB200_THROW("outputs must be set before rocalVerify");
    if (!owns(t)) RB200_THROW("rocalSetOutputs: not a tensor of this context");
    t->is_output = true;
    if (std::find(_output_order.begin(), _output_order.end(), t->id) == _output_order.end()) _output_order.push_back(t->id);
}

void Pipeline::verify() {
    if (_verified) RB200_THROW("rocalVerify was already called");
    if (_source < 0) RB200_THROW("the graph has no input source");
    if (_bbox_crop && _tensors[_source]->is_output) RB200_THROW("a source cut by rocalRandomBBoxCrop cannot be a graph output");
    RB200_CUDA(cudaSetDevice(_gpu_id));
    plan();
    _slots.resize(_depth);
    size_t table_bytes = std::max<size_t>(1, _steps.size()) * _batch * 64;
    for (auto& t : _tensors) {
        if (t->is_source) {
            if (t->is_output) t->materialized = false;   // the source is exposed through the input arena
            continue;
        }
        if (!t->materialized) continue;
        if (t->is_output) {
            t->ring.resize(_depth, nullptr);
            for (size_t s = 0; s < _depth; s++) RB200_CUDA(cudaMalloc(&t->ring[s], t->data_size()));
        } else {
            RB200_CUDA(cudaMalloc(&t->scratch, t->data_size()));
        }
    }
    for (auto& t : _tensors)          // outputs flagged at creation that never went through mark_output
        if (t->is_output && std::find(_output_order.begin(), _output_order.end(), t->id) == _output_order.end())
            _output_order.push_back(t->id);
    for (int id : _output_order) {
        TensorImpl* t = _tensors[(size_t)id].get();
        if (t->is_output && !t->is_source) _output_list.items.push_back(t);
    }
    if (const char* e = std::getenv("RB200_PROFILE")) _profiling = _profiling || std::atoi(e) != 0;
    if (_profiling) {
        _step_timing.clear();
        _step_timing.push_back({"upload", 0.0, 0});
        for (const Step& st : _steps) _step_timing.push_back({step_name(st), 0.0, 0});
    }
    if (log_level() >= 2) {
        std::fprintf(stderr, "[rb200] plan: batch %zu, %zu launches per batch, ring depth %zu\n", _batch, _steps.size(), _depth);
        for (size_t k = 0; k < _steps.size(); k++) {
            TensorImpl* o = _tensors[_steps[k].out_tensor].get();
            std::fprintf(stderr, "[rb200]   step %zu: %s -> %d x %d, %zu bytes%s\n", k, step_name(_steps[k]).c_str(), o->max_w, o->max_h,
                         (size_t)o->data_size(), o->is_output ? " (output)" : "");
        }
    }
    for (auto& s : _slots) {
        if (_profiling) {
            s.step_ev.resize(_steps.size() + 2, nullptr);
            for (auto& ev : s.step_ev) RB200_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDefault));
        }
        RB200_CUDA(cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming));
        RB200_CUDA(cudaEventCreateWithFlags(&s.consumer_done, cudaEventDisableTiming));
        RB200_CUDA(cudaHostAlloc((void**)&s.h_status, 64, cudaHostAllocMapped));
        *s.h_status = 0;
        RB200_CUDA(cudaHostGetDevicePointer((void**)&s.d_status, s.h_status, 0));
        RB200_CUDA(cudaMalloc(&s.d_tables, table_bytes));
        RB200_CUDA(cudaHostAlloc(&s.h_tables, table_bytes, cudaHostAllocDefault));
        s.rois.assign(_tensors.size(), std::vector<unsigned>());
        s.windows.assign(_nodes.size(), std::vector<unsigned>());
        if (_box_encoder) {
            RB200_CUDA(cudaMalloc((void**)&s.d_enc_boxes, _batch * (size_t)_enc.num_anchors * 4 * sizeof(float)));
            RB200_CUDA(cudaMalloc((void**)&s.d_enc_labels, _batch * (size_t)_enc.num_anchors * sizeof(int)));
        }
        if (_box_matcher) RB200_CUDA(cudaMalloc((void**)&s.d_matches, _batch * (size_t)_match.num_anchors * sizeof(int)));
    }
    for (const Step& st : _steps) {
        if (st.kind != Step::NORMALIZE) continue;
        const Node& nd = _nodes[st.node];
        if (!nd.stat_mean.empty() && !nd.stat_std.empty()) continue;       // nothing is computed
        TensorImpl* out = _tensors[st.out_tensor].get();
        _norm_scratch_bytes = std::max(_norm_scratch_bytes, rb200k_normalize_scratch_bytes((int)_batch, out->max_w, out->max_h, nd.axis_mask));
    }
    if (_norm_scratch_bytes) RB200_CUDA(cudaMalloc(&_norm_scratch, _norm_scratch_bytes));
    for (int k = 0; k < 2; k++) RB200_CUDA(cudaEventCreateWithFlags(&_arena_free[k], cudaEventDisableTiming));
    if (_box_matcher) {
        RB200_CUDA(cudaMalloc((void**)&_d_match_anchors, _match_anchors.size() * sizeof(float)));
        RB200_CUDA(cudaMemcpy(_d_match_anchors, _match_anchors.data(), _match_anchors.size() * sizeof(float), cudaMemcpyHostToDevice));
        _match.anchors = _d_match_anchors;
        _matches_t.reset(new TensorImpl(this, -3, (int)_batch, 1, _match.num_anchors, ROCAL_INT32, ROCAL_NHWC, false, false));
        _matches_t->custom_dims = {_batch, (size_t)_match.num_anchors};
        _match_list.items = {_matches_t.get()};
    }
    if (_box_encoder || _box_matcher) {
        _box_capacity = _batch * 64;
        RB200_CUDA(cudaMalloc((void**)&_d_boxes, _box_capacity * 4 * sizeof(float)));
        RB200_CUDA(cudaMalloc((void**)&_d_labels, _box_capacity * sizeof(int)));
        RB200_CUDA(cudaMalloc((void**)&_d_offsets, (_batch + 1) * sizeof(int)));
        RB200_CUDA(cudaHostAlloc(&_h_box_stage, _box_capacity * 5 * sizeof(float) + (_batch + 1) * sizeof(int), cudaHostAllocDefault));
    }
    if (_box_encoder) {
        RB200_CUDA(cudaMalloc((void**)&_d_anchors, _anchors.size() * sizeof(float)));
        RB200_CUDA(cudaMemcpy(_d_anchors, _anchors.data(), _anchors.size() * sizeof(float), cudaMemcpyHostToDevice));
        _enc.anchors = _d_anchors;
        _enc_boxes_t.reset(new TensorImpl(this, -1, (int)_batch, 4, _enc.num_anchors, ROCAL_FP32, ROCAL_NHWC, false, false));
        _enc_labels_t.reset(new TensorImpl(this, -2, (int)_batch, 1, _enc.num_anchors, ROCAL_INT32, ROCAL_NHWC, false, false));
        _enc_boxes_t->custom_dims = {_batch, (size_t)_enc.num_anchors, 4};
        _enc_labels_t->custom_dims = {_batch, (size_t)_enc.num_anchors};
        _enc_list_boxes.items = {_enc_boxes_t.get()};
        _enc_list_labels.items = {_enc_labels_t.get()};
        _enc_meta.lists = {&_enc_list_labels, &_enc_list_boxes};
    }
    // Parameters that feed per-sample tables keep one value per sample.
    for (auto& nd : _nodes) {
        for (auto* p : {nd.mirror, nd.flip_h, nd.flip_v})
            if (p) p->create_array((unsigned)_batch);
        for (auto* p : nd.color)
            if (p) p->create_array((unsigned)_batch);
        if (nd.angle) nd.angle->create_array((unsigned)_batch);
    }
    _verified = true;
    _worker = std::thread(&Pipeline::worker_loop, this);
    top_up();
}

// ------------------------------------------------------------------------------------------
// Feeding
// ------------------------------------------------------------------------------------------

void Pipeline::stage_boxes(const float* ltrb, const int* labels, const int* counts, size_t n) {
    if (n != _batch) RB200_THROW("rb200_feed_boxes: expected one count per sample of the batch");
    size_t total = 0;
    for (size_t i = 0; i < n; i++) {
        if (counts[i] < 0) RB200_THROW("rb200_feed_boxes: negative box count");
        total += (size_t)counts[i];
    }
    _staged.boxes.assign(ltrb, ltrb + total * 4);
    _staged.labels.assign(labels, labels + total);
    _staged.counts.assign(counts, counts + n);
    _staged.has_boxes = true;
}

void Pipeline::stage_anchors(TensorImpl* t, const float* ax, const float* ay, size_t n) {
    if (!owns(t) || t->producer < 0 || _nodes[t->producer].kind != NodeKind::CROP_MIRROR_NORMALIZE)
        RB200_THROW("rb200_set_crop_anchors: the tensor is not the output of a CropMirrorNormalize call");
    if (n != _batch) RB200_THROW("rb200_set_crop_anchors: expected one anchor pair per sample");
    _staged.anchors_x.emplace_back(t->producer, std::vector<float>(ax, ax + n));
    _staged.anchors_y.emplace_back(t->producer, std::vector<float>(ay, ay + n));
}

void Pipeline::stage_affine(TensorImpl* t, const float* m6, size_t n) {
    if (!owns(t) || t->producer < 0 || _nodes[t->producer].kind != NodeKind::WARP_AFFINE)
        RB200_THROW("rb200_set_affine: the tensor is not the output of a WarpAffine call");
    if (n != _batch) RB200_THROW("rb200_set_affine: expected one table per sample");
    _staged.affines.emplace_back(t->producer, std::vector<float>(m6, m6 + n * 6));
}

void Pipeline::feed(InputBatch&& b) {
    if (!_verified) RB200_THROW("rocalVerify must be called before feeding input");
    if (b.n != _batch) RB200_THROW("a fed batch must hold exactly batch_size samples (got " + std::to_string(b.n) + ")");
    TensorImpl* src = _tensors[_source].get();
    if (b.kind == InputBatch::SLOTS) {
        for (size_t i = 0; i < b.n; i++) {
            if (!b.bufs[i]) RB200_THROW("null input buffer");
            unsigned x = b.roi[i * 4], y = b.roi[i * 4 + 1], w = b.roi[i * 4 + 2], h = b.roi[i * 4 + 3];
            if (w == 0 || h == 0 || x + w > b.max_w || y + h > b.max_h)
                RB200_THROW("input ROI of sample " + std::to_string(i) + " is empty or exceeds max_width x max_height");
        }
    } else if (b.kind == InputBatch::ENCODED) {
        if (b.paths.empty())
            for (size_t i = 0; i < b.n; i++)
                if (!b.bufs[i] || b.enc_sizes[i] == 0) RB200_THROW("encoded image " + std::to_string(i) + " is empty");
    } else {
        if (!b.arena) RB200_THROW("null input arena");
        for (size_t i = 0; i < b.n; i++) {
            const auto& d = b.descs[i];
            if (d.width == 0 || d.height == 0 || d.stride < d.width * 3 ||
                d.offset + (uint64_t)(d.height - 1) * d.stride + (uint64_t)d.width * 3 > b.arena_bytes)
                RB200_THROW("image descriptor " + std::to_string(i) + " is empty or exceeds the arena");
            if (d.width > (unsigned)src->max_w || d.height > (unsigned)src->max_h)
                RB200_THROW("image " + std::to_string(i) + " exceeds the source's max_width x max_height");
        }
    }
    b.has_boxes = _staged.has_boxes;
    b.boxes = std::move(_staged.boxes);
    b.labels = std::move(_staged.labels);
    b.counts = std::move(_staged.counts);
    b.anchors_x = std::move(_staged.anchors_x);
    b.anchors_y = std::move(_staged.anchors_y);
    b.affines = std::move(_staged.affines);
    _staged = InputBatch();
    {
        std::lock_guard<std::mutex> lk(_m);
        _queue.push_back(std::move(b));
        _in_flight++;
    }
    _cv_work.notify_one();
}

size_t Pipeline::remaining() {
    std::lock_guard<std::mutex> lk(_m);
    size_t r = _in_flight * _batch;
    if (_files) r += _files->batches_left() * _batch;
    return r;
}

// ------------------------------------------------------------------------------------------
// Worker: upload -> tables -> launches -> event
// ------------------------------------------------------------------------------------------

void Pipeline::worker_loop() {
    cudaSetDevice(_gpu_id);
    for (;;) {
        InputBatch b;
        size_t slot_idx;
        {
            std::unique_lock<std::mutex> lk(_m);
            _cv_work.wait(lk, [&] { return _stop || (!_queue.empty() && _slots[_write].state == Slot::FREE); });
            if (_stop) return;
            b = std::move(_queue.front());
            _queue.pop_front();
            slot_idx = _write;
        }
        Slot& s = _slots[slot_idx];
        s.error.clear();
        try {
            process(b, s, (int)slot_idx);
        } catch (const std::exception& e) {
            s.error = e.what();
        }
        {
            std::lock_guard<std::mutex> lk(_m);
            s.state = Slot::READY;
            _write = (_write + 1) % _depth;
        }
        _cv_ready.notify_all();
    }
}

void Pipeline::ensure_arena(int which, size_t bytes) {
    if (_arena_cap[which] >= bytes) return;
    if (_arena[which]) {
        RB200_CUDA(cudaStreamSynchronize(_stream));
        RB200_CUDA(cudaFree(_arena[which]));
        _arena[which] = nullptr;
        _arena_cap[which] = 0;
    }
    size_t cap = bytes + bytes / 8 + 4096;
    RB200_CUDA(cudaMalloc(&_arena[which], cap));
    _arena_cap[which] = cap;
}

void Pipeline::sync_copy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind) {
    RB200_CUDA(cudaSetDevice(_gpu_id));
    unsigned long long t0 = now_us();
    RB200_CUDA(cudaMemcpy(dst, src, bytes, kind));
    _t_transfer += now_us() - t0;
}

// Seeded SSD random crop. The reference's node draws from std::random_device and its width/height
// draws are shadowed (source/augmentations/node_ssd_random_crop.cpp:90-136), so the window is produced
// by this sampler instead, with the node's structure: an option out of 7 minimum-IoU settings
// (option 0 = keep the whole image), width and height factors in [0.3, 1], aspect ratio in [0.5, 2],
// uniform position, every box IoU >= the option, at least one box centre inside.
void Pipeline::ssd_crop(Node& nd, const std::vector<int>& in_w, const std::vector<int>& in_h, Slot& s) {
    static const float kMinIou[7] = {0.0f, 0.1f, 0.3f, 0.5f, 0.45f, 0.35f, 0.0f};
    size_t n = in_w.size();
    nd.crop.x1v.assign(n, 0);
    nd.crop.y1v.assign(n, 0);
    nd.crop.cwv.resize(n);
    nd.crop.chv.resize(n);
    unsigned base_seed = ParameterFactory::instance().get_seed();
    unsigned batch_id = nd.batch_counter++;
    size_t box0 = 0;
    std::vector<float> crops(n * 4);
    for (size_t i = 0; i < n; i++) {
        std::mt19937 gen(base_seed * 2654435761u + batch_id * 40503u + (unsigned)i);
        auto uni = [&](float lo, float hi) {
            return (float)(((double)gen() / 4294967295.0) * ((double)hi - (double)lo) + (double)lo);
        };
        int nb = s.counts.empty() ? 0 : s.counts[i];
        const float* bb = s.boxes.data() + box0 * 4;
        float l = 0.f, t = 0.f, r = 1.f, b = 1.f;
        for (int round = 0; round < 64; round++) {
            int option = (int)(gen() % 7u);
            if (option == 0) break;
            float min_iou = kMinIou[option];
            bool found = false;
            for (int a = 0; a < nd.ssd_attempts && !found; a++) {
                float w = uni(0.3f, 1.0f), h = uni(0.3f, 1.0f);
                float ar = w / h;
                if (ar < 0.5f || ar > 2.0f) continue;
                float x = uni(0.0f, 1.0f - w), y = uni(0.0f, 1.0f - h);
                float cl = x, ct = y, cr = x + w, cb = y + h;
                bool ok = true;
                int centres = 0;
                for (int j = 0; j < nb && ok; j++) {
                    const float* q = bb + j * 4;
                    float xa = std::max(q[0], cl), ya = std::max(q[1], ct), xb = std::min(q[2], cr), yb = std::min(q[3], cb);
                    float inter = std::max(0.f, xb - xa) * std::max(0.f, yb - ya);
                    float a1 = (q[2] - q[0]) * (q[3] - q[1]), a2 = (cr - cl) * (cb - ct);
                    float iou = inter / (a1 + a2 - inter);
                    if (iou < min_iou) ok = false;
                    float xc = 0.5f * (q[0] + q[2]), yc = 0.5f * (q[1] + q[3]);
                    if (xc > cl && xc < cr && yc > ct && yc < cb) centres++;
                }
                if (!ok || (nb > 0 && centres == 0)) continue;
                l = cl; t = ct; r = cr; b = cb;
                found = true;
            }
            if (found) break;
        }
        crops[i * 4] = l; crops[i * 4 + 1] = t; crops[i * 4 + 2] = r; crops[i * 4 + 3] = b;
        unsigned W = (unsigned)in_w[i], H = (unsigned)in_h[i];
        unsigned x1 = (unsigned)(l * W), y1 = (unsigned)(t * H);
        unsigned cw = (unsigned)((r - l) * W), ch = (unsigned)((b - t) * H);
        if (x1 >= W) x1 = W - 1;
        if (y1 >= H) y1 = H - 1;
        nd.crop.x1v[i] = x1;
        nd.crop.y1v[i] = y1;
        nd.crop.cwv[i] = std::max(1u, std::min(cw, W - x1));
        nd.crop.chv[i] = std::max(1u, std::min(ch, H - y1));
        box0 += (size_t)nb;
    }
    transform_boxes_window(s, nd.crop.x1v, nd.crop.y1v, nd.crop.cwv, nd.crop.chv, in_w, in_h, true);
}

// Boxes follow a crop window, in normalized ltrb (a box times the image size is the reference's pixel box).
// by_centre = true: the rule of the SSD crop, update_random_bbox_meta_data (source/meta_data/bounding_box_graph.cpp:
// 98-110) — a box is kept when its centre lies strictly inside the window; a sample left without boxes gets one
// empty box with label 0. by_centre = false: the rule of the Crop / CropMirrorNormalize / ResizeCropMirror meta nodes
// (source/meta_data/meta_node_crop.cpp:59-78, meta_node_crop_mirror_normalize.cpp:53-90,
// meta_node_resize_crop_mirror.cpp:66-100) — a box is kept when at least a quarter of its area lies in the window
// (MetaNode::BBoxIntersectionOverUnion without is_iou, threshold 0.25, include/meta_data/meta_node.h:39-58); a sample
// left without boxes gets the whole window with label 0. Kept boxes are clipped to the window and re-normalised to it.
void Pipeline::transform_boxes_window(Slot& s, const std::vector<unsigned>& x1, const std::vector<unsigned>& y1,
                                      const std::vector<unsigned>& cw, const std::vector<unsigned>& ch,
                                      const std::vector<int>& in_w, const std::vector<int>& in_h, bool by_centre) {
    if (s.counts.empty()) return;
    std::vector<float> nb;
    std::vector<int> nl, nc(s.counts.size(), 0);
    size_t box0 = 0;
    for (size_t i = 0; i < s.counts.size(); i++) {
        float l = (float)x1[i] / in_w[i], t = (float)y1[i] / in_h[i];
        float r = (float)(x1[i] + cw[i]) / in_w[i], b = (float)(y1[i] + ch[i]) / in_h[i];
        float w = r - l, h = b - t;
        for (int j = 0; j < s.counts[i]; j++) {
            const float* q = s.boxes.data() + (box0 + j) * 4;
            bool keep;
            if (by_centre) {
                float xc = 0.5f * (q[0] + q[2]), yc = 0.5f * (q[1] + q[3]);
                keep = xc > l && xc < r && yc > t && yc < b;
            } else {
                float xa = std::max(q[0], l), ya = std::max(q[1], t), xb = std::min(q[2], r), yb = std::min(q[3], b);
                float inter = std::max(0.f, xb - xa) * std::max(0.f, yb - ya);
                float area = (q[3] - q[1]) * (q[2] - q[0]);
                keep = inter / area >= 0.25f;      // 0/0 (an empty box) is NaN and drops the box, as in the reference
            }
            if (keep) {
                nb.push_back((std::max(q[0], l) - l) / w);
                nb.push_back((std::max(q[1], t) - t) / h);
                nb.push_back((std::min(q[2], r) - l) / w);
                nb.push_back((std::min(q[3], b) - t) / h);
                nl.push_back(s.labels[box0 + j]);
                nc[i]++;
            }
        }
        if (nc[i] == 0) {
            if (by_centre) nb.insert(nb.end(), {0.f, 0.f, 0.f, 0.f});
            else nb.insert(nb.end(), {0.f, 0.f, 1.f, 1.f});
            nl.push_back(0);
            nc[i] = 1;
        }
        box0 += (size_t)s.counts[i];
    }
    s.boxes.swap(nb);
    s.labels.swap(nl);
    s.counts.swap(nc);
}

// Horizontal mirror of normalized ltrb boxes (meta_node_flip.cpp:40-55, meta_node_crop_mirror_normalize.cpp:53-74);
// `vertical` mirrors top and bottom instead (the v_flip branch of meta_node_flip.cpp:56-60).
void Pipeline::mirror_boxes(Slot& s, const std::vector<int>& flags, bool vertical) {
    if (s.counts.empty()) return;
    size_t box0 = 0;
    const int lo = vertical ? 1 : 0, hi = vertical ? 3 : 2;
    for (size_t i = 0; i < s.counts.size(); i++) {
        if (flags[i]) {
            for (int j = 0; j < s.counts[i]; j++) {
                float* q = s.boxes.data() + (box0 + j) * 4;
                float l = 1.0f - q[hi], r = 1.0f - q[lo];
                q[lo] = l;
                q[hi] = r;
            }
        }
        box0 += (size_t)s.counts[i];
    }
}

// Boxes behind a Rotate operator: RotateMetaNode::update_parameters (source/meta_data/meta_node_rotate.cpp:27-103),
// in the pixel coordinates it works in. The four corners of a box are rotated about the image centres (source
// centre = roi size / 2 in float, destination centre = size / 2 in integer arithmetic, as there), the new box is
// their bounding box - with its left and top edge taken as min(0, .), as the node writes it, so every kept box starts
// at the image's corner after the clip -, kept when at least a quarter of it lies in the destination image, clipped to
// it; a sample left without boxes gets the whole destination image with label 0. Results are re-normalised to the
// destination size.
void Pipeline::rotate_boxes(Slot& s, const std::vector<float>& angle_deg, const std::vector<int>& in_w, const std::vector<int>& in_h,
                            int dst_w, int dst_h) {
    if (s.counts.empty()) return;
    std::vector<float> nb;
    std::vector<int> nl, nc(s.counts.size(), 0);
    size_t box0 = 0;
    const float W = (float)dst_w, H = (float)dst_h;
    for (size_t i = 0; i < s.counts.size(); i++) {
        const float radian = (float)((double)angle_deg[i] * 3.14159265 / 180);
        const float r0 = (float)std::cos((double)radian), r1 = (float)std::sin((double)radian), r2 = -1 * r1, r3 = r0;
        const float dcx = (float)(dst_w / 2), dcy = (float)(dst_h / 2);
        const float scx = (float)in_w[i] / 2, scy = (float)in_h[i] / 2;
        for (int j = 0; j < s.counts[i]; j++) {
            const float* q = s.boxes.data() + (box0 + j) * 4;
            const float x = q[0] * in_w[i], y = q[1] * in_h[i];
            const float bw = q[2] * in_w[i] - x, bh = q[3] * in_h[i] - y;
            const float x1 = (r0 * (x - scx)) + (r1 * (y - scy)) + dcx, y1 = (r2 * (x - scx)) + (r3 * (y - scy)) + dcy;
            const float x2 = (r0 * ((x + bw) - scx)) + (r1 * (y - scy)) + dcx, y2 = (r2 * ((x + bw) - scx)) + (r3 * (y - scy)) + dcy;
            const float x3 = (r0 * (x - scx)) + (r1 * ((y + bh) - scy)) + dcx, y3 = (r2 * (x - scx)) + (r3 * ((y + bh) - scy)) + dcy;
            const float x4 = (r0 * ((x + bw) - scx)) + (r1 * ((y + bh) - scy)) + dcx,
                        y4 = (r2 * ((x + bw) - scx)) + (r3 * ((y + bh) - scy)) + dcy;
            float l = std::min(0.0f, std::min(x1, std::min(x2, std::min(x3, x4))));
            float t = std::min(0.0f, std::min(y1, std::min(y2, std::min(y3, y4))));
            float r = std::max(x1, std::max(x2, std::max(x3, x4)));
            float b = std::max(y1, std::max(y2, std::max(y3, y4)));
            const float xa = std::max(l, 0.f), ya = std::max(t, 0.f), xb = std::min(r, W), yb = std::min(b, H);
            const float inter = std::max(0.f, xb - xa) * std::max(0.f, yb - ya);
            const float area = (b - t) * (r - l);
            if (inter / area >= 0.25f) {
                nb.push_back(std::max(0.f, l) / W);
                nb.push_back(std::max(0.f, t) / H);
                nb.push_back(std::min(W, r) / W);
                nb.push_back(std::min(H, b) / H);
                nl.push_back(s.labels[box0 + j]);
                nc[i]++;
            }
        }
        if (nc[i] == 0) {
            nb.insert(nb.end(), {0.f, 0.f, 1.f, 1.f});
            nl.push_back(0);
            nc[i] = 1;
        }
        box0 += (size_t)s.counts[i];
    }
    s.boxes.swap(nb);
    s.labels.swap(nl);
    s.counts.swap(nc);
}

void Pipeline::update_nodes(const InputBatch& b, Slot& s) {
    size_t n = _batch;
    for (auto& a : b.anchors_x) _nodes[a.first].crop.next_anchor_x = a.second;
    for (auto& a : b.anchors_y) _nodes[a.first].crop.next_anchor_y = a.second;
    for (auto& a : b.affines) _nodes[a.first].next_affine = a.second;
    ParameterFactory::instance().renew_parameters();
    for (auto& nd : _nodes) {
        TensorImpl* in = _tensors[nd.in].get();
        TensorImpl* out = _tensors[nd.out].get();
        auto int_array = [&](Parameter<int>* p, std::vector<int>& dst) {
            dst.assign(n, 0);
            if (!p) return;
            const auto& a = p->array();
            for (size_t i = 0; i < n; i++) dst[i] = a.size() == n ? a[i] : p->get();
        };
        switch (nd.kind) {
            case NodeKind::RESIZE:
            case NodeKind::RESIZE_MIRROR_NORMALIZE: {
                nd.dst_w.resize(n);
                nd.dst_h.resize(n);
                for (size_t i = 0; i < n; i++) {
                    unsigned w, h;
                    resize_target((unsigned)in->roi_w[i], (unsigned)in->roi_h[i], nd.dest_w, nd.dest_h, nd.scaling_mode,
                                  nd.max_w, nd.max_h, w, h);
                    nd.dst_w[i] = (int)std::max(1u, std::min(w, (unsigned)out->max_w));
                    nd.dst_h[i] = (int)std::max(1u, std::min(h, (unsigned)out->max_h));
                }
                out->roi_w = nd.dst_w;
                out->roi_h = nd.dst_h;
                if (nd.kind == NodeKind::RESIZE_MIRROR_NORMALIZE) {
                    std::vector<int> m;
                    int_array(nd.mirror, m);
                    mirror_boxes(s, m);
                }
                break;
            }
            case NodeKind::RESIZE_CROP_MIRROR: {
                nd.crop.update(in->roi_w, in->roi_h);
                nd.dst_w.assign(n, (int)nd.dest_w);
                nd.dst_h.assign(n, (int)nd.dest_h);
                out->roi_w = nd.dst_w;
                out->roi_h = nd.dst_h;
                transform_boxes_window(s, nd.crop.x1v, nd.crop.y1v, nd.crop.cwv, nd.crop.chv, in->roi_w, in->roi_h, false);
                std::vector<int> m;
                int_array(nd.mirror, m);
                mirror_boxes(s, m);
                break;
            }
            case NodeKind::CROP:
            case NodeKind::CROP_MIRROR_NORMALIZE: {
                nd.crop.update(in->roi_w, in->roi_h);
                for (size_t i = 0; i < n; i++) {
                    out->roi_w[i] = (int)std::min(nd.crop.cwv[i], (unsigned)out->max_w);
                    out->roi_h[i] = (int)std::min(nd.crop.chv[i], (unsigned)out->max_h);
                }
                transform_boxes_window(s, nd.crop.x1v, nd.crop.y1v, nd.crop.cwv, nd.crop.chv, in->roi_w, in->roi_h, false);
                if (nd.kind == NodeKind::CROP_MIRROR_NORMALIZE) {
                    std::vector<int> m;
                    int_array(nd.mirror, m);
                    mirror_boxes(s, m);
                }
                break;
            }
            case NodeKind::SSD_RANDOM_CROP: {
                ssd_crop(nd, in->roi_w, in->roi_h, s);
                for (size_t i = 0; i < n; i++) {
                    out->roi_w[i] = (int)std::min(nd.crop.cwv[i], (unsigned)out->max_w);
                    out->roi_h[i] = (int)std::min(nd.crop.chv[i], (unsigned)out->max_h);
                }
                break;
            }
            case NodeKind::FLIP: {
                out->roi_w = in->roi_w;
                out->roi_h = in->roi_h;
                std::vector<int> m;
                int_array(nd.flip_h, m);
                mirror_boxes(s, m);
                int_array(nd.flip_v, m);
                mirror_boxes(s, m, true);
                break;
            }
            case NodeKind::WARP_AFFINE: {
                if (!s.counts.empty()) RB200_THROW("bounding boxes cannot follow a WarpAffine operator (no metadata rule for it)");
                nd.affine_v.resize(n * 6);
                if (nd.next_affine.size() == n * 6) {
                    nd.affine_v = nd.next_affine;
                    nd.next_affine.clear();
                } else {
                    // x0, y0, x1, y1, o0, o1: the packing of WarpAffineNode::update_affine_array
                    // (node_warp_affine.cpp:67-75), one renewal per sample and coefficient.
                    static const int order[6] = {0, 2, 1, 3, 4, 5};
                    for (size_t i = 0; i < n; i++)
                        for (int k = 0; k < 6; k++) {
                            Parameter<float>* p = nd.affine[order[k]];
                            p->renew();
                            nd.affine_v[i * 6 + k] = p->get();
                        }
                }
                for (size_t i = 0; i < n; i++) {
                    out->roi_w[i] = out->max_w;
                    out->roi_h[i] = out->max_h;
                }
                break;
            }
            case NodeKind::ROTATE: {
                nd.affine_v.resize(n * 6);
                const auto& a = nd.angle->array();
                if (!s.counts.empty()) {
                    std::vector<float> deg(n);
                    for (size_t i = 0; i < n; i++) deg[i] = a.size() == n ? a[i] : nd.angle->get();
                    rotate_boxes(s, deg, in->roi_w, in->roi_h, out->max_w, out->max_h);
                }
                for (size_t i = 0; i < n; i++) {
                    float deg = a.size() == n ? a[i] : nd.angle->get();
                    float rad = deg * (float)(M_PI / 180.0);
                    float c = (float)std::cos((double)rad), sn = (float)std::sin((double)rad);
                    float* m = &nd.affine_v[i * 6];
                    m[0] = c; m[1] = -sn; m[2] = sn; m[3] = c; m[4] = 0.f; m[5] = 0.f;
                    out->roi_w[i] = out->max_w;
                    out->roi_h[i] = out->max_h;
                }
                break;
            }
            default:   // colour operators keep the geometry
                out->roi_w = in->roi_w;
                out->roi_h = in->roi_h;
        }
    }
}

// The rectangle of source image i that the kernels of this batch can read, from the step tables that
// were just built: every step that consumes the source tensor contributes the bounding box of its taps
// (resample: crop window of the resized image mapped back through the ratio, with a margin that covers the
// half-pixel offset, both taps and rounding; pointwise: its window). Steps whose reach is not a simple
// rectangle (affine gathers), or a source that is itself an output, ask for the whole image.
bool Pipeline::source_footprint(const uint8_t* h_tab, size_t i, int W, int H, int& x0, int& y0, int& x1, int& y1) const {
    const size_t n = _batch;
    if (_tensors[_source]->is_output) return false;
    int fx0 = W, fy0 = H, fx1 = -1, fy1 = -1;
    bool any = false;
    for (size_t k = 0; k < _steps.size(); k++) {
        const Step& st = _steps[k];
        if (st.in2_tensor == _source) return false;      // a blend reads the whole second image
        if (st.in_tensor != _source) continue;
        int ax0, ay0, ax1, ay1;
        if (st.kind == Step::RESAMPLE) {
            const rb200_resample_sample& q = reinterpret_cast<const rb200_resample_sample*>(h_tab + k * n * 64)[i];
            if (q.dst_w <= 0 || q.dst_h <= 0 || q.roi_w <= 0 || q.roi_h <= 0) return false;
            const double rx = (double)q.roi_w / q.dst_w, ry = (double)q.roi_h / q.dst_h;
            // reach of the filter on each side of the mapped position: one tap for bilinear, the radius
            // B * max(ratio, 1) for the generic filters (B = 1 triangular / gaussian, 2 bicubic, 3 lanczos, 0.5 nearest)
            const int interp = _nodes[st.resize].interpolation;
            const bool tri = interp != RB200_INTERP_BILINEAR;
            const double base = interp == RB200_INTERP_BICUBIC ? 2.0 : (interp == RB200_INTERP_LANCZOS ? 3.0 : 1.0);
            const double mx = tri ? base * std::max(rx, 1.0) + 1.0 : 1.0, my = tri ? base * std::max(ry, 1.0) + 1.0 : 1.0;
            ax0 = q.roi_x + (int)std::floor(q.crop_x * rx - mx) - 1;
            ay0 = q.roi_y + (int)std::floor(q.crop_y * ry - my) - 1;
            ax1 = q.roi_x + (int)std::ceil((q.crop_x + q.crop_w) * rx + mx - 1.0) + 2;
            ay1 = q.roi_y + (int)std::ceil((q.crop_y + q.crop_h) * ry + my - 1.0) + 2;
            ax0 = std::max(ax0, q.roi_x); ay0 = std::max(ay0, q.roi_y);
            ax1 = std::min(ax1, q.roi_x + q.roi_w - 1); ay1 = std::min(ay1, q.roi_y + q.roi_h - 1);
        } else if (st.kind == Step::POINTWISE) {
            const rb200_pointwise_sample& q = reinterpret_cast<const rb200_pointwise_sample*>(h_tab + k * n * 64)[i];
            ax0 = q.roi_x; ay0 = q.roi_y; ax1 = q.roi_x + q.roi_w - 1; ay1 = q.roi_y + q.roi_h - 1;
        } else {
            return false;
        }
        fx0 = std::min(fx0, ax0); fy0 = std::min(fy0, ay0);
        fx1 = std::max(fx1, ax1); fy1 = std::max(fy1, ay1);
        any = true;
    }
    if (!any) return false;
    x0 = std::max(fx0, 0); y0 = std::max(fy0, 0);
    x1 = std::min(fx1, W - 1); y1 = std::min(fy1, H - 1);
    return x0 <= x1 && y0 <= y1;
}

// Host -> device copy of the batch's source pixels into arena `a`. Only the footprint rectangle of every
// image travels (one strided copy per image, placed where the whole image would be, so tables and kernels
// do not change); when the footprints add up to nearly everything a ragged arena goes up in one copy.
void Pipeline::upload_sources(InputBatch& b, int a, const uint8_t* h_tab) {
    const size_t n = _batch;
    TensorImpl* src = _tensors[_source].get();
    std::vector<int> rect(n * 4);
    size_t need = 0, full = 0;
    for (size_t i = 0; i < n; i++) {
        const int W = src->roi_w[i], H = src->roi_h[i];
        int x0 = 0, y0 = 0, x1 = W - 1, y1 = H - 1;
        if (_upload_mode != UPLOAD_WHOLE) source_footprint(h_tab, i, W, H, x0, y0, x1, y1);
        rect[i * 4] = x0; rect[i * 4 + 1] = y0; rect[i * 4 + 2] = x1; rect[i * 4 + 3] = y1;
        need += (size_t)(x1 - x0 + 1) * (y1 - y0 + 1) * 3;
        full += (size_t)W * H * 3;
    }
    if (a < 0) {
        // zero copy: the one kernel that consumes the source fetches its rows itself, each row once - every row of the
        // window for ratios below 2, the two tap rows of every output row above - as whole 16-byte granules around the
        // span its taps cover (about 15 bytes of rounding per row)
        size_t pulled = 0;
        for (size_t k = 0; k < _steps.size(); k++) {
            const Step& st = _steps[k];
            if (st.in_tensor != _source) continue;
            const TensorImpl* ot = _tensors[st.out_tensor].get();
            for (size_t i = 0; i < n; i++) {
                if (st.kind == Step::RESAMPLE) {
                    const rb200_resample_sample& q = reinterpret_cast<const rb200_resample_sample*>(h_tab + k * n * 64)[i];
                    const double rx = (double)q.roi_w / q.dst_w, ry = (double)q.roi_h / q.dst_h;
                    const int out_rows = std::min(q.crop_h, ot->max_h), out_cols = std::min(q.crop_w, ot->max_w);
                    const long rows = std::min<long>(std::min<long>(2L * out_rows, (long)std::ceil(out_rows * ry) + 1), q.roi_h);
                    const long span = std::min<long>((long)std::ceil(out_cols * rx) + 2, q.roi_w);
                    pulled += (size_t)rows * (size_t)(span * 3 + 15);
                } else {
                    const rb200_pointwise_sample& q = reinterpret_cast<const rb200_pointwise_sample*>(h_tab + k * n * 64)[i];
                    pulled += (size_t)std::min(q.roi_h, ot->max_h) * (size_t)(std::min(q.roi_w, ot->max_w) * 3 + 15);
                }
            }
        }
        _h2d_bytes += pulled ? pulled : need;
        return;
    }
    uint8_t* dst = (uint8_t*)_arena[a];
    if (b.kind == InputBatch::RAGGED && (double)need > 0.9 * (double)b.arena_bytes) {
        RB200_CUDA(cudaMemcpyAsync(dst, b.arena, b.arena_bytes, cudaMemcpyHostToDevice, _stream));
        _h2d_bytes += b.arena_bytes;
        return;
    }
    for (size_t i = 0; i < n; i++) {
        const int x0 = rect[i * 4], y0 = rect[i * 4 + 1], x1 = rect[i * 4 + 2], y1 = rect[i * 4 + 3];
        if (x1 < x0 || y1 < y0) continue;
        const size_t dpitch = _src_views[i].stride;
        const size_t width = (size_t)(x1 - x0 + 1) * 3, height = (size_t)(y1 - y0 + 1);
        uint8_t* d = dst + _src_views[i].offset + (size_t)y0 * dpitch + (size_t)x0 * 3;
        const uint8_t* h;
        size_t spitch;
        if (b.kind == InputBatch::RAGGED) {
            spitch = dpitch;
            h = (const uint8_t*)b.arena + _src_views[i].offset + (size_t)y0 * spitch + (size_t)x0 * 3;
        } else {
            spitch = (size_t)b.max_w * 3;
            h = b.bufs[i] + ((size_t)(b.roi[i * 4 + 1] + y0) * b.max_w + b.roi[i * 4] + x0) * 3;
        }
        RB200_CUDA(cudaMemcpy2DAsync(d, dpitch, h, spitch, width, height, cudaMemcpyHostToDevice, _stream));
        _h2d_bytes += width * height;
    }
}

void Pipeline::process(InputBatch& b, Slot& s, int slot_idx) {
    const size_t n = _batch;
    TensorImpl* src = _tensors[_source].get();
    unsigned long long t0 = now_us();
    if (s.consumer_pending) {
        // a consumer may still be reading this slot's buffers on its own stream (consumer_fence)
        RB200_CUDA(cudaStreamWaitEvent(_stream, s.consumer_done, 0));
        RB200_CUDA(cudaStreamWaitEvent(_meta_stream, s.consumer_done, 0));
        s.consumer_pending = false;
    }

    // ---- 1. input: device views of the n source images (the upload itself follows the tables) ----
    _src_views.resize(n);
    s.decoder_windows.clear();
    s.bbox_crop_windows.clear();
    _whole_w.assign(n, 0);
    _whole_h.assign(n, 0);
    size_t bbox_box0 = 0;
    if (_bbox_crop) {
        if (!b.has_boxes || b.counts.size() != n)
            RB200_THROW("rocalRandomBBoxCrop: the batch carries no bounding boxes (feed them, or use a COCO source)");
        s.decoder_windows.resize(n * 4);
        s.bbox_crop_windows.resize(n * 4);
    }
    // random bbox crop: sample i's window inside its W x H image, in pixels as the reference's fused decoder rounds it
    // (FusedCropTJDecoder::decode, source/decoders/image/fused_crop_decoder.cpp:76-85), kept inside the image
    auto bbox_window = [&](size_t i, int W, int H) -> CropRect {
        float* f = &s.bbox_crop_windows[i * 4];
        _bbox_crop->window(b.boxes.data() + bbox_box0 * 4, b.counts[i], W, f);
        bbox_box0 += (size_t)b.counts[i];
        CropRect win;
        win.x = (unsigned)std::min<long>(std::lround(f[0] * W), W - 1);
        win.y = (unsigned)std::min<long>(std::lround(f[1] * H), H - 1);
        win.w = (unsigned)std::max<long>(1, std::min<long>(std::lround(f[2] * W), W - (long)win.x));
        win.h = (unsigned)std::max<long>(1, std::min<long>(std::lround(f[3] * H), H - (long)win.y));
        unsigned* dw = &s.decoder_windows[i * 4];
        dw[0] = win.x; dw[1] = win.y; dw[2] = win.w; dw[3] = win.h;
        return win;
    };
    const bool host_input = !(b.kind == InputBatch::RAGGED && b.mem_kind == RB200_MEM_DEVICE);
    int arena_used = -1;
    if (b.kind == InputBatch::RAGGED) {
        for (size_t i = 0; i < n; i++) {
            _src_views[i] = {b.descs[i].offset, b.descs[i].stride};
            src->roi_w[i] = _whole_w[i] = (int)b.descs[i].width;
            src->roi_h[i] = _whole_h[i] = (int)b.descs[i].height;
            if (_bbox_crop) {
                const CropRect win = bbox_window(i, _whole_w[i], _whole_h[i]);
                _src_views[i].offset += (size_t)win.y * b.descs[i].stride + (size_t)win.x * 3;
                src->roi_w[i] = (int)win.w;
                src->roi_h[i] = (int)win.h;
            }
        }
        if (!host_input) _src_base = (const uint8_t*)b.arena;
    } else if (b.kind == InputBatch::ENCODED) {
        // JPEG streams: sizes from the headers, then one batched decode into the packed arena (below)
        if (!b.paths.empty()) {
            b.enc_owned.resize(n);
            b.bufs.resize(n);
            b.enc_sizes.resize(n);
            for (size_t i = 0; i < n; i++) {
                read_file(b.paths[i], b.enc_owned[i]);
                b.bufs[i] = b.enc_owned[i].data();
                b.enc_sizes[i] = b.enc_owned[i].size();
            }
        }
        _jpeg.init();
        size_t total = 0;
        _decode_off.resize(n);
        _decode_h.resize(n);
        // behind rocalRandomBBoxCrop the fused decoder cuts the box-aware windows, not its own random ones
        // (FusedCropTJDecoder::decode, fused_crop_decoder.cpp:76-85: the bbox coordinates win when there are any)
        if (_crop_dec && !_bbox_crop) {
            s.decoder_batch_seed = _crop_dec->next_batch(n);
            s.decoder_windows.resize(n * 4);
        }
        for (size_t i = 0; i < n; i++) {
            int w = 0, h = 0;
            _jpeg.image_size(b.bufs[i], b.enc_sizes[i], w, h);
            if (w <= 0 || h <= 0 || w > src->max_w || h > src->max_h)
                RB200_THROW("decoded image " + std::to_string(i) + " (" + std::to_string(w) + "x" + std::to_string(h) +
                            ") is empty or exceeds the source's max_width x max_height");
            _decode_off[i] = total;
            _decode_h[i] = h;
            _src_views[i] = {total, (uint32_t)w * 3};
            src->roi_w[i] = _whole_w[i] = w;
            src->roi_h[i] = _whole_h[i] = h;
            if (_crop_dec || _bbox_crop) {
                // the whole image is decoded; the graph sees the window as its source image (a view into it)
                CropRect win;
                if (_crop_dec && !_bbox_crop) {
                    win = _crop_dec->window(h, w, i);
                    unsigned* dw = &s.decoder_windows[i * 4];
                    dw[0] = win.x; dw[1] = win.y; dw[2] = win.w; dw[3] = win.h;
                } else {
                    win = bbox_window(i, w, h);
                }
                _src_views[i].offset = total + (size_t)win.y * w * 3 + (size_t)win.x * 3;
                src->roi_w[i] = (int)win.w;
                src->roi_h[i] = (int)win.h;
            }
            total += ((size_t)w * h * 3 + 255) & ~(size_t)255;
        }
        b.arena_bytes = total + 256;
    } else {
        size_t total = 0;
        for (size_t i = 0; i < n; i++) {
            _whole_w[i] = (int)b.roi[i * 4 + 2];
            _whole_h[i] = (int)b.roi[i * 4 + 3];
            if (_bbox_crop) {          // only the window is uploaded: the slot's region of interest becomes the window
                const CropRect win = bbox_window(i, _whole_w[i], _whole_h[i]);
                b.roi[i * 4] += win.x; b.roi[i * 4 + 1] += win.y;
                b.roi[i * 4 + 2] = win.w; b.roi[i * 4 + 3] = win.h;
            }
            unsigned w = b.roi[i * 4 + 2], h = b.roi[i * 4 + 3];
            _src_views[i] = {total, w * 3};
            src->roi_w[i] = (int)w;
            src->roi_h[i] = (int)h;
            total += ((size_t)w * h * 3 + 255) & ~(size_t)255;
        }
        b.arena_bytes = total + 256;
    }
    s.source_wh.resize(n * 2);
    for (size_t i = 0; i < n; i++) {
        s.source_wh[i * 2] = src->roi_w[i];
        s.source_wh[i * 2 + 1] = src->roi_h[i];
    }
    if (!s.decoder_windows.empty())   // the views show the windows; report the images they were cut from
        for (size_t i = 0; i < n; i++) {
            s.source_wh[i * 2] = _whole_w[i];
            s.source_wh[i * 2 + 1] = _whole_h[i];
        }
    // Pinned host input that exactly one staging kernel consumes is not uploaded at all: the kernel's bulk
    // copies read the tap rows straight from host memory, so only the bytes the batch needs cross the link.
    bool zero_copy = false;
    if (host_input && _upload_mode == UPLOAD_ZERO_COPY && b.kind == InputBatch::RAGGED &&
        b.mem_kind == RB200_MEM_HOST_PINNED && !src->is_output) {
        int consumers = 0;
        bool gather = false;
        for (const Step& st : _steps) {
            if (st.in2_tensor == _source) consumers += 2;    // a second-source reader rules zero-copy out
            if (st.in_tensor == _source) {
                consumers++;
                // kernels that fetch every tap on its own (affine gathers, the triangular filter) would cross
                // the link once per tap
                gather = gather || st.kind == Step::WARP || st.kind == Step::NORMALIZE || st.kind == Step::TRANSPOSE ||
                         (st.kind == Step::RESAMPLE && _nodes[st.resize].interpolation != RB200_INTERP_BILINEAR);
            }
        }
        if (consumers == 1 && !gather) {
            void* dp = nullptr;
            if (cudaHostGetDevicePointer(&dp, const_cast<void*>(b.arena), 0) == cudaSuccess && dp) {
                _src_base = (const uint8_t*)dp;
                zero_copy = true;
            } else {
                cudaGetLastError();   // not mapped into the device's address space: upload instead
            }
        }
    }
    if (host_input && !zero_copy) {
        arena_used = _arena_next;
        _arena_next ^= 1;
        RB200_CUDA(cudaEventSynchronize(_arena_free[arena_used]));
        ensure_arena(arena_used, b.arena_bytes);
        _src_base = (const uint8_t*)_arena[arena_used];
    }
    _t_load += now_us() - t0;
    t0 = now_us();

    // ---- 2. per-sample tables ----
    std::optional<NvtxRange> tables_range;
    tables_range.emplace("rb200 tables");
    s.boxes = b.boxes;
    s.labels = b.labels;
    s.counts = b.counts;
    s.file_labels = b.file_labels;
    s.names = b.names;
    s.padded = b.padded;
    if (_bbox_crop) {
        // the boxes follow the window by the centre rule (BoundingBoxGraph::update_random_bbox_meta_data)
        std::vector<unsigned> wx(n), wy(n), ww(n), wh(n);
        for (size_t i = 0; i < n; i++) {
            wx[i] = s.decoder_windows[i * 4]; wy[i] = s.decoder_windows[i * 4 + 1];
            ww[i] = s.decoder_windows[i * 4 + 2]; wh[i] = s.decoder_windows[i * 4 + 3];
        }
        transform_boxes_window(s, wx, wy, ww, wh, _whole_w, _whole_h, true);
    }
    update_nodes(b, s);
    ParameterFactory::instance().snapshot(n, s.int_params, s.float_params);

    auto view_of = [&](int tensor_id, size_t i, const uint8_t*& base) -> SampleView {
        TensorImpl* t = _tensors[tensor_id].get();
        if (t->is_source) {
            base = _src_base;
            return _src_views[i];
        }
        base = (const uint8_t*)(t->is_output ? t->ring[slot_idx] : t->scratch);
        return {(uint64_t)i * t->max_h * t->max_w * 3, (uint32_t)t->max_w * 3};
    };

    uint8_t* h_tab = (uint8_t*)s.h_tables;
    const unsigned long long probe_cycles = _probe_wait_cycles.load();
    const int probe_skip = _probe_skip_row.load();
    for (size_t k = 0; k < _steps.size(); k++) {
        const Step& st = _steps[k];
        TensorImpl* in = _tensors[st.in_tensor].get();
        const uint8_t* base = nullptr;
        if (st.kind == Step::RESAMPLE) {
            auto* tab = reinterpret_cast<rb200_resample_sample*>(h_tab + k * n * 64);
            const Node& R = _nodes[st.resize];
            for (size_t i = 0; i < n; i++) {
                SampleView v = view_of(st.in_tensor, i, base);
                rb200_resample_sample& q = tab[i];
                std::memset(&q, 0, sizeof(q));
                q.src_offset = v.offset;
                q.src_stride = v.stride;
                if (st.pre_crop >= 0) {
                    const CropSpec& c = _nodes[st.pre_crop].crop;
                    q.roi_x = (int)c.x1v[i]; q.roi_y = (int)c.y1v[i]; q.roi_w = (int)c.cwv[i]; q.roi_h = (int)c.chv[i];
                } else if (R.kind == NodeKind::RESIZE_CROP_MIRROR) {
                    q.roi_x = (int)R.crop.x1v[i]; q.roi_y = (int)R.crop.y1v[i];
                    q.roi_w = (int)R.crop.cwv[i]; q.roi_h = (int)R.crop.chv[i];
                } else {
                    q.roi_w = in->roi_w[i];
                    q.roi_h = in->roi_h[i];
                }
                q.dst_w = R.dst_w[i];
                q.dst_h = R.dst_h[i];
                if (st.post >= 0) {
                    const Node& C = _nodes[st.post];
                    q.crop_x = (int)C.crop.x1v[i]; q.crop_y = (int)C.crop.y1v[i];
                    q.crop_w = (int)C.crop.cwv[i]; q.crop_h = (int)C.crop.chv[i];
                    const auto& ma = C.mirror->array();
                    q.mirror = (ma.size() == n ? ma[i] : C.mirror->get()) ? 1 : 0;
                } else {
                    q.crop_w = q.dst_w;
                    q.crop_h = q.dst_h;
                    if (R.mirror) {
                        const auto& ma = R.mirror->array();
                        q.mirror = (ma.size() == n ? ma[i] : R.mirror->get()) ? 1 : 0;
                    }
                }
            }
        } else if (st.kind == Step::NORMALIZE || st.kind == Step::TRANSPOSE) {
            auto* tab = reinterpret_cast<rb200_pointwise_sample*>(h_tab + k * n * 64);
            for (size_t i = 0; i < n; i++) {
                SampleView v = view_of(st.in_tensor, i, base);
                rb200_pointwise_sample& q = tab[i];
                std::memset(&q, 0, sizeof(q));
                q.src_offset = v.offset;
                q.src_stride = v.stride;
                q.roi_w = in->roi_w[i];
                q.roi_h = in->roi_h[i];
            }
        } else if (st.kind == Step::POINTWISE) {
            auto* tab = reinterpret_cast<rb200_pointwise_sample*>(h_tab + k * n * 64);
            for (size_t i = 0; i < n; i++) {
                SampleView v = view_of(st.in_tensor, i, base);
                rb200_pointwise_sample& q = tab[i];
                std::memset(&q, 0, sizeof(q));
                q.src_offset = v.offset;
                q.src_stride = v.stride;
                q.roi_w = in->roi_w[i];
                q.roi_h = in->roi_h[i];
                q.alpha = 1.f; q.sat = 1.f;
                if (st.window >= 0) {
                    const Node& W = _nodes[st.window];
                    q.roi_x = (int)W.crop.x1v[i]; q.roi_y = (int)W.crop.y1v[i];
                    q.roi_w = (int)W.crop.cwv[i]; q.roi_h = (int)W.crop.chv[i];
                    if (W.mirror) {
                        const auto& ma = W.mirror->array();
                        q.flip_h = (ma.size() == n ? ma[i] : W.mirror->get()) ? 1 : 0;
                    }
                }
                if (st.flip >= 0) {
                    const Node& F = _nodes[st.flip];
                    const auto& ha = F.flip_h->array();
                    const auto& va = F.flip_v->array();
                    q.flip_h = (ha.size() == n ? ha[i] : F.flip_h->get()) ? 1 : 0;
                    q.flip_v = (va.size() == n ? va[i] : F.flip_v->get()) ? 1 : 0;
                }
                if (st.color >= 0) {
                    const Node& C = _nodes[st.color];
                    auto val = [&](int slot, float dflt) {
                        Parameter<float>* p = C.color[slot];
                        if (!p) return dflt;
                        const auto& a = p->array();
                        return a.size() == n ? a[i] : p->get();
                    };
                    switch (C.kind) {
                        case NodeKind::BRIGHTNESS: q.alpha = val(0, 1.f); q.beta = val(1, 0.f); break;
                        // exposure: x * 2^factor; colour temperature: R + adjustment, B - adjustment (brightness
                        // operator with a tilted offset); gamma: its own operator with alpha = gamma
                        case NodeKind::EXPOSURE: q.alpha = std::exp2(val(0, 0.f)); q.beta = 0.f; break;
                        case NodeKind::GAMMA: q.alpha = val(0, 1.f); break;
                        case NodeKind::BLEND: {
                            // the second source's view, as an offset from this step's base pointer
                            const uint8_t* base2 = nullptr;
                            const SampleView v2 = view_of(st.in2_tensor, i, base2);
                            const uint64_t rel = (uint64_t)(uintptr_t)(base2 + v2.offset) - (uint64_t)(uintptr_t)base;
                            q.src2_offset_lo = (uint32_t)rel;
                            q.src2_offset_hi = (uint32_t)(rel >> 32);
                            q.src2_stride = v2.stride;
                            q.alpha = val(0, 0.5f);
                            break;
                        }
                        case NodeKind::COLOR_TEMP: {
                            const auto& a = C.adjustment->array();
                            q.alpha = 1.f; q.beta = 0.f;
                            q.hue = (float)(a.size() == n ? a[i] : C.adjustment->get());
                            break;
                        }
                        case NodeKind::CONTRAST: q.alpha = val(0, 1.f); q.beta = val(1, 0.f); break;
                        case NodeKind::HUE: q.hue = val(2, 0.f); break;
                        case NodeKind::SATURATION: q.sat = val(3, 1.f); break;
                        default: q.alpha = val(0, 1.f); q.beta = val(1, 0.f); q.hue = val(2, 0.f); q.sat = val(3, 1.f);
                    }
                }
            }
        } else {
            auto* tab = reinterpret_cast<rb200_warp_sample*>(h_tab + k * n * 64);
            const Node& W = _nodes[st.warp];
            TensorImpl* out = _tensors[st.out_tensor].get();
            for (size_t i = 0; i < n; i++) {
                SampleView v = view_of(st.in_tensor, i, base);
                rb200_warp_sample& q = tab[i];
                std::memset(&q, 0, sizeof(q));
                q.src_offset = v.offset;
                q.src_stride = v.stride;
                q.src_w = in->roi_w[i];
                q.src_h = in->roi_h[i];
                for (int c = 0; c < 6; c++) q.m[c] = W.affine_v[i * 6 + c];
                q.dst_w = out->max_w;
                q.dst_h = out->max_h;
            }
        }
    }
    tables_range.reset();
    s.step_ev_valid = false;
    if (_profiling) RB200_CUDA(cudaEventRecord(s.step_ev[0], _stream));
    if (b.kind == InputBatch::ENCODED) {
        NvtxRange range("rb200 decode");
        unsigned long long tl = now_us();
        _jpeg_dst.resize(n);
        _jpeg_pitch.resize(n);
        size_t enc = 0;
        for (size_t i = 0; i < n; i++) {
            _jpeg_dst[i] = (unsigned char*)_arena[arena_used] + _decode_off[i];
            _jpeg_pitch[i] = _src_views[i].stride;
            enc += b.enc_sizes[i];
        }
        _jpeg.decode_batch(b.bufs.data(), b.enc_sizes.data(), (int)n, _jpeg_dst.data(), _jpeg_pitch.data(), _stream);
        _h2d_bytes += enc;
        _t_decode += now_us() - tl;
    } else if (host_input) {
        NvtxRange range("rb200 upload");
        unsigned long long tl = now_us();
        upload_sources(b, arena_used, (const uint8_t*)s.h_tables);
        _t_load += now_us() - tl;
    }
    if (!_steps.empty()) {
        RB200_CUDA(cudaMemcpyAsync(s.d_tables, s.h_tables, _steps.size() * n * 64, cudaMemcpyHostToDevice, _stream));
        _h2d_bytes += _steps.size() * n * 64;
    }

    if (_profiling) RB200_CUDA(cudaEventRecord(s.step_ev[1], _stream));

    // ---- 3. launches ----
    NvtxRange launch_range("rb200 launches");
    for (size_t k = 0; k < _steps.size(); k++) {
        const Step& st = _steps[k];
        TensorImpl* out = _tensors[st.out_tensor].get();
        const uint8_t* base = nullptr;
        view_of(st.in_tensor, 0, base);
        void* out_ptr = out->is_output ? out->ring[slot_idx] : out->scratch;
        const void* d_tab = (const uint8_t*)s.d_tables + k * n * 64;
        const void* h_tabk = h_tab + k * n * 64;
        int out_dtype = out->dtype == ROCAL_FP32 ? RB200_FP32 : (out->dtype == ROCAL_FP16 ? RB200_FP16 : RB200_UINT8);
        int out_layout = out->lay == ROCAL_NCHW ? RB200_NCHW : RB200_NHWC;
        // sizes of what the launch reads and writes (checked by the bounds-checking build of the kernels)
        TensorImpl* in_t = _tensors[st.in_tensor].get();
        const uint64_t in_bytes = in_t->is_source ? (uint64_t)b.arena_bytes : (uint64_t)in_t->data_size();
        const uint64_t out_bytes = (uint64_t)out->data_size();
        int rc = 0;
        if (st.kind == Step::RESAMPLE) {
            rb200_resample_params p{};
            p.out = out_ptr;
            p.out_w = out->max_w;
            p.out_h = out->max_h;
            p.out_dtype = out_dtype;
            p.out_layout = out_layout;
            const Node* norm = st.post >= 0 ? &_nodes[st.post] : &_nodes[st.resize];
            p.normalize = norm->normalize ? 1 : 0;
            for (int c = 0; c < 3; c++) { p.mul[c] = norm->mul[c]; p.add[c] = norm->add[c]; }
            // A fixed-size output (crop or stretch target) is fully defined, padding zeroed; a
            // plain resize into its max-shape tensor defines only the ROI, as the reference does.
            p.fill_padding = (st.post >= 0 || _nodes[st.resize].kind != NodeKind::RESIZE) ? 1 : 0;
            p.interpolation = _nodes[st.resize].interpolation;
            // a source read in place from pinned host memory is streamed row by row, every row once
            p.path = (zero_copy && in_t->is_source) ? RB200_RESAMPLE_PATH_ROWS : RB200_RESAMPLE_PATH_PAIRS;
            p.status = s.d_status;
            p.arena_bytes = in_bytes;
            p.out_bytes = out_bytes;
            rc = probe_cycles ? rb200k_resample_probe(base, (const rb200_resample_sample*)d_tab, (const rb200_resample_sample*)h_tabk,
                                                      (int)n, &p, _stream, probe_cycles, probe_skip)
                              : rb200k_resample(base, (const rb200_resample_sample*)d_tab, (const rb200_resample_sample*)h_tabk, (int)n, &p, _stream);
        } else if (st.kind == Step::POINTWISE) {
            rb200_pointwise_params p{};
            p.out = out_ptr;
            p.out_w = out->max_w;
            p.out_h = out->max_h;
            p.out_dtype = out_dtype;
            p.out_layout = out_layout;
            p.color_op = RB200_COLOR_NONE;
            if (st.color >= 0) {
                NodeKind ck = _nodes[st.color].kind;
                p.color_op = (ck == NodeKind::BRIGHTNESS || ck == NodeKind::EXPOSURE || ck == NodeKind::COLOR_TEMP) ? RB200_COLOR_BRIGHTNESS
                             : ck == NodeKind::CONTRAST ? RB200_COLOR_CONTRAST
                             : ck == NodeKind::GAMMA    ? RB200_COLOR_GAMMA
                             : ck == NodeKind::BLEND    ? RB200_COLOR_BLEND : RB200_COLOR_TWIST;
            }
            for (int c = 0; c < 3; c++) { p.mul[c] = 1.f; p.add[c] = 0.f; }
            if (st.window >= 0 && _nodes[st.window].normalize) {
                p.normalize = 1;
                for (int c = 0; c < 3; c++) { p.mul[c] = _nodes[st.window].mul[c]; p.add[c] = _nodes[st.window].add[c]; }
            }
            p.fill_padding = (st.window >= 0) ? 1 : 0;
            p.arith = _arith;
            p.status = s.d_status;
            p.arena_bytes = in_bytes;
            p.out_bytes = out_bytes;
            rc = probe_cycles ? rb200k_pointwise_probe(base, (const rb200_pointwise_sample*)d_tab, (const rb200_pointwise_sample*)h_tabk,
                                                       (int)n, &p, _stream, probe_cycles, probe_skip)
                              : rb200k_pointwise(base, (const rb200_pointwise_sample*)d_tab, (const rb200_pointwise_sample*)h_tabk, (int)n, &p, _stream);
        } else if (st.kind == Step::NORMALIZE) {
            const Node& nd = _nodes[st.node];
            rb200_normalize_params p{};
            p.out = out_ptr;
            p.out_w = out->max_w;
            p.out_h = out->max_h;
            p.out_dtype = out_dtype;
            p.axis_mask = nd.axis_mask;
            p.compute_mean = nd.stat_mean.empty() ? 1 : 0;
            p.compute_stddev = nd.stat_std.empty() ? 1 : 0;
            p.fill_padding = 1;
            for (int c = 0; c < 3; c++) {
                p.mean[c] = nd.stat_mean.empty() ? 0.f : nd.stat_mean[std::min<size_t>(c, nd.stat_mean.size() - 1)];
                p.stddev[c] = nd.stat_std.empty() ? 1.f : nd.stat_std[std::min<size_t>(c, nd.stat_std.size() - 1)];
            }
            p.scale = nd.stat_scale;
            p.shift = nd.stat_shift;
            p.arena_bytes = in_bytes;
            p.out_bytes = out_bytes;
            rc = rb200k_normalize(base, (const rb200_pointwise_sample*)d_tab, (const rb200_pointwise_sample*)h_tabk, (int)n, &p,
                                  _norm_scratch, _norm_scratch_bytes, _stream);
        } else if (st.kind == Step::TRANSPOSE) {
            const Node& nd = _nodes[st.node];
            const int32_t od[3] = {(int32_t)out->custom_dims[1], (int32_t)out->custom_dims[2], (int32_t)out->custom_dims[3]};
            RB200_CUDA(cudaMemsetAsync(out_ptr, 0, out->data_size(), _stream));
            rc = rb200k_transpose(base, (const rb200_pointwise_sample*)d_tab, (int)n, nd.perm, (uint8_t*)out_ptr, od, _stream);
        } else {
            rb200_warp_params p{};
            p.out = out_ptr;
            p.out_w = out->max_w;
            p.out_h = out->max_h;
            p.fill_padding = 1;
            p.status = s.d_status;
            p.arena_bytes = in_bytes;
            p.out_bytes = out_bytes;
            rc = rb200k_warp_affine(base, (const rb200_warp_sample*)d_tab, (int)n, &p, _stream);
        }
        if (rc != 0) RB200_THROW(rb200k_last_error());
        if (_profiling) RB200_CUDA(cudaEventRecord(s.step_ev[k + 2], _stream));
    }
    s.step_ev_valid = _profiling;
    if (arena_used >= 0) RB200_CUDA(cudaEventRecord(_arena_free[arena_used], _stream));

    // ---- 4. box encoder / box IoU matcher ----
    if (_box_encoder || _box_matcher) {
        if (s.counts.size() != n) RB200_THROW("the box encoder / matcher needs boxes for every batch (rb200_feed_boxes)");
        size_t total = s.labels.size();
        int max_boxes = 1;
        for (int c : s.counts) max_boxes = std::max(max_boxes, c);
        if (total > _box_capacity) {
            RB200_CUDA(cudaStreamSynchronize(_meta_stream));
            cudaFree(_d_boxes);
            cudaFree(_d_labels);
            cudaFreeHost(_h_box_stage);
            _box_capacity = total * 2;
            RB200_CUDA(cudaMalloc((void**)&_d_boxes, _box_capacity * 4 * sizeof(float)));
            RB200_CUDA(cudaMalloc((void**)&_d_labels, _box_capacity * sizeof(int)));
            RB200_CUDA(cudaHostAlloc(&_h_box_stage, _box_capacity * 5 * sizeof(float) + (_batch + 1) * sizeof(int), cudaHostAllocDefault));
        } else {
            // the staging block is reused: the previous batch's three copies out of it must be done
            RB200_CUDA(cudaEventSynchronize(_box_stage_free));
        }
        float* hb = (float*)_h_box_stage;
        int* hl = (int*)(hb + _box_capacity * 4);
        int* ho = hl + _box_capacity;
        std::memcpy(hb, s.boxes.data(), total * 4 * sizeof(float));
        std::memcpy(hl, s.labels.data(), total * sizeof(int));
        ho[0] = 0;
        for (size_t i = 0; i < n; i++) ho[i + 1] = ho[i] + s.counts[i];
        RB200_CUDA(cudaMemcpyAsync(_d_boxes, hb, total * 4 * sizeof(float), cudaMemcpyHostToDevice, _meta_stream));
        RB200_CUDA(cudaMemcpyAsync(_d_labels, hl, total * sizeof(int), cudaMemcpyHostToDevice, _meta_stream));
        RB200_CUDA(cudaMemcpyAsync(_d_offsets, ho, (n + 1) * sizeof(int), cudaMemcpyHostToDevice, _meta_stream));
        RB200_CUDA(cudaEventRecord(_box_stage_free, _meta_stream));
        _h2d_bytes += total * 20 + (n + 1) * sizeof(int);
        if (_box_encoder) {
            int rc = rb200k_box_encode(_d_boxes, _d_labels, _d_offsets, (int)n, max_boxes, &_enc, s.d_enc_boxes, s.d_enc_labels, _meta_stream);
            if (rc != 0) RB200_THROW(rb200k_last_error());
        }
        if (_box_matcher) {
            int rc = rb200k_box_iou_match(_d_boxes, _d_offsets, (int)n, max_boxes, &_match, s.d_matches, _meta_stream);
            if (rc != 0) RB200_THROW(rb200k_last_error());
        }
        RB200_CUDA(cudaEventRecord(_meta_done, _meta_stream));
        RB200_CUDA(cudaStreamWaitEvent(_stream, _meta_done, 0));
    }

    // ---- 5. snapshot of the ROIs the user will see, completion event ----
    for (auto& t : _tensors) {
        auto& r = s.rois[t->id];
        r.resize(n * 4);
        for (size_t i = 0; i < n; i++) {
            r[i * 4] = 0; r[i * 4 + 1] = 0;
            r[i * 4 + 2] = (unsigned)t->roi_w[i];
            r[i * 4 + 3] = (unsigned)t->roi_h[i];
        }
    }
    for (size_t k = 0; k < _nodes.size(); k++) {
        const CropSpec& c = _nodes[k].crop;
        auto& w = s.windows[k];
        w.clear();
        if (c.x1v.size() != n) continue;
        w.resize(n * 4);
        for (size_t i = 0; i < n; i++) {
            w[i * 4] = c.x1v[i]; w[i * 4 + 1] = c.y1v[i]; w[i * 4 + 2] = c.cwv[i]; w[i * 4 + 3] = c.chv[i];
        }
    }
    s.n = n;
    RB200_CUDA(cudaEventRecord(s.done, _stream));
    _t_process += now_us() - t0;
}

// The buffers of the held batch go back to the ring at the next run(); work that a consumer queued on its own stream
// (a training step reading the zero-copy outputs) may still be pending then. The event recorded here makes the
// worker's streams wait for that work before the slot is written again - no host synchronisation.
void Pipeline::consumer_fence(void* consumer_stream) {
    if (_held < 0) return;
    Slot& s = _slots[_held];
    RB200_CUDA(cudaSetDevice(_gpu_id));
    RB200_CUDA(cudaEventRecord(s.consumer_done, (cudaStream_t)consumer_stream));
    s.consumer_pending = true;
}

void Pipeline::set_arithmetic(int mode) {
    if (mode != RB200_ARITH_EXACT && mode != RB200_ARITH_FAST) RB200_THROW("arithmetic mode must be 0 (exact) or 1 (fast)");
    _arith = mode;
}

void Pipeline::set_wait_probe(unsigned long long wait_cycles, int skip_row) {
    _probe_wait_cycles.store(wait_cycles);
    _probe_skip_row.store(wait_cycles ? skip_row : -1);
}

// ------------------------------------------------------------------------------------------
// run(): hand the next finished batch to the user (MasterGraph::run, master_graph.cpp:193-223)
// ------------------------------------------------------------------------------------------

void Pipeline::run() {
    if (!_verified) RB200_THROW("rocalVerify must be called before rocalRun");
    size_t idx;
    {
        // the previous batch goes back first, so that the folder reader can refill its slot
        std::lock_guard<std::mutex> lk(_m);
        if (_held >= 0) {
            _slots[_held].state = Slot::FREE;
            _held = -1;
            _cv_work.notify_all();
        }
    }
    top_up();
    {
        std::unique_lock<std::mutex> lk(_m);
        if (_held >= 0) {
            _slots[_held].state = Slot::FREE;
            _held = -1;
            _cv_work.notify_all();
        }
        if (_in_flight == 0) RB200_THROW(_files ? "rocalRun: the file source is exhausted (rocalResetLoaders starts the next epoch)"
                                                : "rocalRun: no input batch has been fed");
        _cv_ready.wait(lk, [&] { return _stop || _slots[_read].state == Slot::READY; });
        if (_stop) RB200_THROW("the context is shutting down");
        idx = _read;
        _read = (_read + 1) % _depth;
        _slots[idx].state = Slot::HELD;
        _held = (int)idx;
        _in_flight--;
    }
    Slot& s = _slots[idx];
    if (!s.error.empty()) RB200_THROW(s.error);
    RB200_CUDA(cudaSetDevice(_gpu_id));
    unsigned long long t0 = now_us();
    RB200_CUDA(cudaEventSynchronize(s.done));
    _t_process += now_us() - t0;
    if (s.step_ev_valid) collect_step_timing(s);
    if (const int st = *static_cast<volatile int*>(s.h_status)) {
        *s.h_status = 0;
        if (st == 2)    // bounds-checking build of the kernels
            RB200_THROW("rocalRun: a kernel of this batch found a sample outside its source arena and did not read it; the batch's "
                        "outputs are incomplete");
        // a kernel of this batch gave up on a bounded wait for its source rows and left its output incomplete
        RB200_THROW("rocalRun: a kernel of this batch gave up waiting for its staged source rows; the batch's outputs are incomplete");
    }
    for (auto& t : _tensors) {
        if (t->is_output && !t->is_source) t->current = t->ring[idx];
        t->user_roi = s.rois[t->id];
    }
    if (_box_encoder) {
        _enc_boxes_t->current = s.d_enc_boxes;
        _enc_labels_t->current = s.d_enc_labels;
    }
    if (_box_matcher) _matches_t->current = s.d_matches;
    refresh_box_views();
}

// Per-sample host tensors over the boxes of the held batch: [count_i][4] float32 ltrb and [count_i] int32
// (MasterGraph::bbox_meta_data / labels_meta_data, master_graph.cpp).
void Pipeline::refresh_box_views() {
    _bbox_t.clear();
    _bbox_label_t.clear();
    _bbox_list.items.clear();
    _bbox_label_list.items.clear();
    if (_held < 0) return;
    Slot& s = _slots[_held];
    if (s.counts.size() != _batch) return;
    size_t at = 0;
    for (size_t i = 0; i < _batch; i++) {
        const size_t c = (size_t)s.counts[i];
        std::unique_ptr<TensorImpl> b(new TensorImpl(this, -10, 1, 4, (int)c, ROCAL_FP32, ROCAL_NHWC, false, false));
        b->custom_dims = {c, 4};
        b->host_mem = true;
        b->current = c ? (void*)(s.boxes.data() + at * 4) : nullptr;
        std::unique_ptr<TensorImpl> l(new TensorImpl(this, -11, 1, 1, (int)c, ROCAL_INT32, ROCAL_NHWC, false, false));
        l->custom_dims = {c};
        l->host_mem = true;
        l->current = c ? (void*)(s.labels.data() + at) : nullptr;
        _bbox_list.items.push_back(b.get());
        _bbox_label_list.items.push_back(l.get());
        _bbox_t.push_back(std::move(b));
        _bbox_label_t.push_back(std::move(l));
        at += c;
    }
}

unsigned Pipeline::bounding_box_count() {
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    if (_slots[_held].counts.size() != _batch) RB200_THROW("No label has been loaded for this output image");
    return (unsigned)_slots[_held].labels.size();
}

TensorListImpl* Pipeline::bounding_box_cords() {
    if (_held < 0 || _bbox_list.items.empty()) return nullptr;
    return &_bbox_list;
}

TensorListImpl* Pipeline::bounding_box_labels() {
    if (_held < 0 || _bbox_label_list.items.empty()) return nullptr;
    return &_bbox_label_list;
}

TensorListImpl* Pipeline::matched_indices() {
    if (!_box_matcher || _held < 0) return nullptr;
    return &_match_list;
}

void Pipeline::matches(int** dev, size_t* num_anchors) {
    if (!_box_matcher) RB200_THROW("no box IoU matcher in this graph");
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    *dev = _slots[_held].d_matches;
    *num_anchors = (size_t)_match.num_anchors;
}

MetaListImpl* Pipeline::encoded_meta() {
    if (!_box_encoder || _held < 0) return nullptr;
    return &_enc_meta;
}

void Pipeline::encoded(float** boxes, int** labels, size_t* num_anchors) {
    if (!_box_encoder) RB200_THROW("no box encoder in this graph");
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    *boxes = _slots[_held].d_enc_boxes;
    *labels = _slots[_held].d_enc_labels;
    *num_anchors = (size_t)_enc.num_anchors;
}

void Pipeline::copy_encoded(float* boxes, int* labels) {
    float* db;
    int* dl;
    size_t a;
    encoded(&db, &dl, &a);
    sync_copy(boxes, db, _batch * a * 4 * sizeof(float), cudaMemcpyDeviceToHost);
    sync_copy(labels, dl, _batch * a * sizeof(int), cudaMemcpyDeviceToHost);
}

void Pipeline::current_boxes(std::vector<float>& ltrb, std::vector<int>& labels, std::vector<int>& counts) {
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    ltrb = _slots[_held].boxes;
    labels = _slots[_held].labels;
    counts = _slots[_held].counts;
}

void Pipeline::crop_windows(TensorImpl* t, unsigned* xywh) {
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    if (!owns(t) || t->producer < 0) RB200_THROW("the tensor is not the output of a crop-type operator");
    int node = t->producer;
    if (_slots[_held].windows[node].empty()) {
        // CropResize / ROIResize: the window belongs to the internal crop node in front of the resize
        TensorImpl* in = _tensors[_nodes[node].in].get();
        if (in->producer >= 0 && !in->is_output && !_slots[_held].windows[in->producer].empty()) node = in->producer;
    }
    if (_slots[_held].windows[node].empty()) RB200_THROW("the tensor is not the output of a crop-type operator");
    const auto& w = _slots[_held].windows[node];
    std::memcpy(xywh, w.data(), w.size() * sizeof(unsigned));
}

// rocalToTensor: first output (uint8 NHWC) -> fp32/fp16 NCHW/NHWC with x*mult+off, optional channel
// reversal (MasterGraph::to_tensor, master_graph.cpp:514-856).
void Pipeline::to_tensor(void* out_ptr, int layout, int dtype, const float* mul, const float* add, bool reverse, int mem_type) {
    if (_held < 0) RB200_THROW("no batch is available yet (call rocalRun first)");
    if (_output_list.items.empty()) RB200_THROW("the graph has no output");
    TensorImpl* t = static_cast<TensorImpl*>(_output_list.items[0]);
    if (t->dtype != ROCAL_UINT8 || t->lay != ROCAL_NHWC) RB200_THROW("rocalToTensor converts a uint8 NHWC output");
    if (dtype != ROCAL_FP32 && dtype != ROCAL_FP16) RB200_THROW("rocalToTensor produces FP32 or FP16");
    RB200_CUDA(cudaSetDevice(_gpu_id));
    size_t n = _batch, e = dtype == ROCAL_FP32 ? 4 : 2;
    size_t bytes = n * t->max_w * t->max_h * 3 * e;
    void* d_out = out_ptr;
    void* tmp = nullptr;
    if (mem_type != ROCAL_MEMCPY_GPU) {
        RB200_CUDA(cudaMalloc(&tmp, bytes));
        d_out = tmp;
    }
    std::vector<rb200_pointwise_sample> tab(n);
    for (size_t i = 0; i < n; i++) {
        std::memset(&tab[i], 0, sizeof(tab[i]));
        tab[i].src_offset = (uint64_t)i * t->max_h * t->max_w * 3;
        tab[i].src_stride = (uint32_t)t->max_w * 3;
        tab[i].roi_w = t->max_w;
        tab[i].roi_h = t->max_h;
        tab[i].alpha = 1.f;
        tab[i].sat = 1.f;
    }
    void* d_tab = nullptr;
    cudaError_t err = cudaMalloc(&d_tab, n * 64);
    if (err == cudaSuccess) err = cudaMemcpy(d_tab, tab.data(), n * 64, cudaMemcpyHostToDevice);
    int rc = 0;
    if (err == cudaSuccess) {
        rb200_pointwise_params p{};
        p.out = d_out;
        p.out_w = t->max_w;
        p.out_h = t->max_h;
        p.out_dtype = dtype == ROCAL_FP32 ? RB200_FP32 : RB200_FP16;
        p.out_layout = layout == ROCAL_NCHW ? RB200_NCHW : RB200_NHWC;
        p.normalize = 1;
        p.reverse_channels = reverse ? 1 : 0;
        for (int c = 0; c < 3; c++) { p.mul[c] = mul[c]; p.add[c] = add[c]; }
        rc = rb200k_pointwise((const uint8_t*)t->current, (const rb200_pointwise_sample*)d_tab, tab.data(), (int)n, &p, _stream);
        if (rc == 0) err = cudaStreamSynchronize(_stream);
        if (rc == 0 && err == cudaSuccess && tmp) err = cudaMemcpy(out_ptr, tmp, bytes, cudaMemcpyDeviceToHost);
    }
    if (d_tab) cudaFree(d_tab);
    if (tmp) cudaFree(tmp);
    if (rc != 0) RB200_THROW(rb200k_last_error());
    if (err != cudaSuccess) RB200_THROW(std::string("rocalToTensor: ") + cudaGetErrorString(err));
}

size_t Pipeline::batch_int_array(const void* core, int* out, size_t n) {
    if (_held < 0 || !out) return 0;
    for (const auto& kv : _slots[_held].int_params)
        if (kv.first == core) {
            const size_t k = std::min(n, kv.second.size());
            std::copy(kv.second.begin(), kv.second.begin() + k, out);
            return k;
        }
    return 0;
}

size_t Pipeline::batch_float_array(const void* core, float* out, size_t n) {
    if (_held < 0 || !out) return 0;
    for (const auto& kv : _slots[_held].float_params)
        if (kv.first == core) {
            const size_t k = std::min(n, kv.second.size());
            std::copy(kv.second.begin(), kv.second.begin() + k, out);
            return k;
        }
    return 0;
}

void Pipeline::set_profiling(bool on) {
    if (_verified) RB200_THROW("profiling must be chosen before rocalVerify");
    _profiling = on;
}

std::string Pipeline::step_name(const Step& st) const {
    switch (st.kind) {
        case Step::RESAMPLE: return "resample";
        case Step::POINTWISE: return "pointwise";
        case Step::NORMALIZE: return "normalize";
        case Step::TRANSPOSE: return "transpose";
        default: return "warp_affine";
    }
}

// The batch's done event has completed, so every event of the slot has: device time between consecutive events.
void Pipeline::collect_step_timing(Slot& s) {
    std::lock_guard<std::mutex> lk(_prof_m);
    for (size_t k = 0; k + 1 < s.step_ev.size() && k < _step_timing.size(); k++) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, s.step_ev[k], s.step_ev[k + 1]) != cudaSuccess) {
            cudaGetLastError();
            continue;
        }
        _step_timing[k].gpu_us += (double)ms * 1000.0;
        _step_timing[k].batches++;
    }
    s.step_ev_valid = false;
}

std::vector<StepTiming> Pipeline::step_timing() {
    std::lock_guard<std::mutex> lk(_prof_m);
    return _step_timing;
}

TimingInfo Pipeline::timing() {
    TimingInfo t;
    t.load_time = _t_load.load();
    t.decode_time = _t_decode.load();
    t.process_time = _t_process.load();
    t.transfer_time = _t_transfer.load();
    return t;
}

void Pipeline::capture_error(const std::string& msg) {
    std::lock_guard<std::mutex> lk(_err_m);
    _error = msg;
    _status = ROCAL_RUNTIME_ERROR;
}

RocalStatus Pipeline::status() {
    std::lock_guard<std::mutex> lk(_err_m);
    return _status;
}

const char* Pipeline::error_message() {
    std::lock_guard<std::mutex> lk(_err_m);
    return _error.c_str();
}

}  // namespace rb200
