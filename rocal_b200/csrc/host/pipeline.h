// Pipeline runtime behind the rocAL API subset: graph of augmentation nodes, fusion into kernel
// launches, per-batch parameter tables, device buffers, ring of output slots, worker thread.
//
// What it stands in for in the reference (paths under rocAL/):
//   Context / MasterGraph        include/pipeline/context.h:29-53, source/pipeline/master_graph.cpp
//   Node::update_node()          source/augmentations/**/node_*.cpp (per-batch tables)
//   RingBuffer                   source/pipeline/ring_buffer.cpp:113-279,360-387
//   DeviceManagerHip             source/device/device_manager_hip.cpp:53-77 (one stream per context)
//   output_routine thread        source/pipeline/master_graph.cpp:950-1050
// There is no OpenVX graph: verify() fuses node chains into the three kernel families of
// rb200_kernels.h and every batch is a handful of launches on one CUDA stream.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "coco_reader.h"
#include "file_source.h"
#include "jpeg_decoder.h"
#include "params.h"
#include "bbox_crop.h"
#include "random_crop_window.h"
#include "rb200.h"
#include "rocal_api.h"

namespace rb200 {

enum class NodeKind {
    RESIZE, RESIZE_CROP_MIRROR, RESIZE_MIRROR_NORMALIZE, CROP, CROP_MIRROR_NORMALIZE, SSD_RANDOM_CROP, FLIP,
    BRIGHTNESS, CONTRAST, HUE, SATURATION, COLOR_TWIST, EXPOSURE, GAMMA, COLOR_TEMP, BLEND, WARP_AFFINE, ROTATE,
    NORMALIZE, TRANSPOSE
};

// Crop window rules of RocalCropParam::fill_crop_dims (source/parameters/parameter_rocal_crop.cpp:49-85) and, for
// RANDOM_AREA, of RocalRandomCropParam::fill_crop_dims (source/parameters/parameter_random_crop.cpp:48-97).
struct CropSpec {
    enum Mode { ABSOLUTE, FIXED_ANCHOR, RANDOM, RANDOM_AREA } mode = ABSOLUTE;
    unsigned crop_w = 0, crop_h = 0, x1 = 0, y1 = 0;
    float anchor_x = 0.5f, anchor_y = 0.5f;
    Parameter<float>*h_factor = nullptr, *w_factor = nullptr, *x_drift = nullptr, *y_drift = nullptr;
    Parameter<float>*area = nullptr, *aspect = nullptr;   // RANDOM_AREA
    std::vector<float> next_anchor_x, next_anchor_y;   // per-sample anchors of the next batch (extension)
    std::vector<unsigned> x1v, y1v, cwv, chv;          // results of the current batch
    void update(const std::vector<int>& in_w, const std::vector<int>& in_h);
};

struct Node {
    NodeKind kind;
    int in = -1, out = -1;
    int in2 = -1;                      // second input tensor (BLEND)
    // resize family
    unsigned dest_w = 0, dest_h = 0, max_w = 0, max_h = 0;
    int scaling_mode = ROCAL_SCALING_MODE_STRETCH;
    int interpolation = RB200_INTERP_BILINEAR;   // resize-type nodes
    std::vector<int> dst_w, dst_h;
    // crop family
    CropSpec crop;
    // mirror / flips
    Parameter<int>*mirror = nullptr, *flip_h = nullptr, *flip_v = nullptr;
    // normalisation tables as the CropMirrorNormalize node builds them
    bool normalize = false;
    float mul[3] = {1, 1, 1}, add[3] = {0, 0, 0};
    // colour: alpha, beta, hue, sat
    Parameter<float>* color[4] = {nullptr, nullptr, nullptr, nullptr};
    Parameter<int>* adjustment = nullptr;   // COLOR_TEMP
    // warp: x0, x1, y0, y1, o0, o1 (API order) or angle
    Parameter<float>* affine[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    Parameter<float>* angle = nullptr;
    std::vector<float> next_affine;    // [n][6] of the next batch (extension)
    std::vector<float> affine_v;       // [n][6] packed {x0,y0,x1,y1,o0,o1}
    // Normalize: axes reduced for computed statistics (bit 0 height, 1 width, 2 channel), given per-channel
    // statistics (empty = computed), scale and shift; Transpose: permutation of (h, w, c)
    int axis_mask = 0;
    std::vector<float> stat_mean, stat_std;
    float stat_scale = 1.f, stat_shift = 0.f;
    int perm[3] = {0, 1, 2};
    int ssd_attempts = 20;
    unsigned batch_counter = 0;        // batches this node has seen (seeds the SSD crop sampler)
    // fusion
    int absorbed_by = -1;              // node index of the consumer this node is fused into
};

class Pipeline;

class TensorImpl : public rocalTensor {
   public:
    TensorImpl(Pipeline* p, int id, int n, int max_w, int max_h, RocalTensorOutputType dt, RocalTensorLayout lay,
               bool is_output, bool is_source);
    void* buffer() override { return current; }
    unsigned copy_data(void* user_buffer, RocalOutputMemType external_mem_type) override;
    unsigned copy_data(void* user_buffer, unsigned x_offset, unsigned y_offset, unsigned max_cols, unsigned max_rows) override;
    unsigned num_of_dims() override { return custom_dims.empty() ? 4u : (unsigned)custom_dims.size(); }
    unsigned batch_size() override { return (unsigned)n; }
    std::vector<size_t> dims() override;
    std::vector<size_t> strides() override;
    RocalTensorLayout layout() override { return lay; }
    RocalTensorBackend backend() override { return host_mem ? ROCAL_CPU : ROCAL_GPU; }
    RocalTensorOutputType data_type() override { return dtype; }
    RocalOutputMemType mem_type() override { return host_mem ? ROCAL_MEMCPY_HOST : ROCAL_MEMCPY_GPU; }
    size_t data_size() override {
        if (!custom_dims.empty()) {
            size_t e = elem_size();
            for (size_t d : custom_dims) e *= d;
            return e;
        }
        return (size_t)n * max_w * max_h * 3 * elem_size();
    }
    RocalROICordsType roi_type() override { return RocalROICordsType::ROCAL_XYWH; }
    size_t get_roi_dims_size() override { return 2; }
    void copy_roi(void* roi_buffer) override;
    std::vector<size_t> shape() override { return dims(); }
    void set_dims(std::vector<size_t>) override {}
    void set_mem_handle(void* b) override { current = b; }
    void set_tensor_layout(RocalTensorLayout l) override { lay = l; }
    uint64_t data_type_size() override { return elem_size(); }
    size_t elem_size() const {
        switch (dtype) {
            case ROCAL_FP32: case ROCAL_INT32: case ROCAL_UINT32: return 4;
            case ROCAL_FP16: case ROCAL_INT16: return 2;
            default: return 1;
        }
    }
    std::vector<size_t> custom_dims;     // non-image tensors (encoded boxes / labels)
    bool host_mem = false;               // metadata tensors (boxes, labels of the batch) live in host memory

    Pipeline* pipe;
    int id, n, max_w, max_h;
    RocalTensorOutputType dtype;
    RocalTensorLayout lay;
    bool is_output, is_source;
    int producer = -1, consumers = 0;
    bool materialized = false;
    std::vector<int> roi_w, roi_h;       // valid extent per sample (worker side, current batch)
    std::vector<void*> ring;             // one device buffer per slot (outputs)
    void* scratch = nullptr;             // device buffer of a non-output intermediate
    void* current = nullptr;             // what the user sees after rocalRun
    std::vector<unsigned> user_roi;      // n x {x,y,w,h} of the batch the user holds
};

class TensorListImpl : public rocalTensorList {
   public:
    uint64_t size() override { return items.size(); }
    rocalTensor* at(size_t i) override { return i < items.size() ? items[i] : nullptr; }
    std::vector<rocalTensor*> items;
};
class MetaListImpl : public rocalListOfTensorList {
   public:
    uint64_t size() override { return lists.size(); }
    rocalTensorList* at(size_t i) override { return i < lists.size() ? lists[i] : nullptr; }
    std::vector<rocalTensorList*> lists;
};

// A device view used as kernel input: base pointer + per-sample offset/stride.
struct SampleView {
    uint64_t offset;
    uint32_t stride;
};

// How host-resident source pixels reach the kernels.
enum UploadMode { UPLOAD_WHOLE = 0, UPLOAD_FOOTPRINT = 1, UPLOAD_ZERO_COPY = 2 };

struct InputBatch {
    enum Kind { SLOTS, RAGGED, ENCODED } kind = SLOTS;
    size_t n = 0;
    std::vector<const unsigned char*> bufs;   // SLOTS
    std::vector<unsigned> roi;                // SLOTS: n x {x,y,w,h}
    unsigned max_w = 0, max_h = 0;
    const void* arena = nullptr;              // RAGGED
    size_t arena_bytes = 0;
    int mem_kind = RB200_MEM_HOST;
    std::vector<rb200_image_desc> descs;
    std::vector<size_t> enc_sizes;                          // ENCODED: byte length of bufs[i]
    std::vector<std::vector<unsigned char>> enc_owned;      // ENCODED from file names: the bytes read at feed time
    std::vector<std::string> paths;                         // ENCODED from the file source: read by the worker
    std::vector<std::string> names;                         // file names reported by rocalGetImageName
    std::vector<int> file_labels;                           // class labels of the file source
    size_t padded = 0;                                      // samples at the end that pad the last batch
    bool has_boxes = false;
    std::vector<float> boxes;                 // ltrb, normalized
    std::vector<int> labels, counts;
    // per-node extensions captured at feed time
    std::vector<std::pair<int, std::vector<float>>> anchors_x, anchors_y, affines;
};

struct Step {
    enum Kind { RESAMPLE, POINTWISE, WARP, NORMALIZE, TRANSPOSE } kind;
    int in_tensor, out_tensor;
    int in2_tensor = -1;                         // POINTWISE with a second source (blend)
    int pre_crop = -1, resize = -1, post = -1;   // RESAMPLE: node indices
    int window = -1, color = -1, flip = -1;      // POINTWISE
    int warp = -1;                               // WARP
    int node = -1;                               // NORMALIZE / TRANSPOSE
};

struct Slot {
    enum State { FREE, READY, HELD } state = FREE;
    cudaEvent_t done = nullptr;
    cudaEvent_t consumer_done = nullptr;   // recorded on a consumer's stream by consumer_fence()
    bool consumer_pending = false;         // the worker must order its streams behind consumer_done before reusing the slot
    int* h_status = nullptr;         // mapped pinned word the kernels of this slot write 1 to when a bounded wait gives up
    int* d_status = nullptr;         // the same word as the device sees it
    void* d_tables = nullptr;        // device copy of all step tables of this slot
    void* h_tables = nullptr;        // pinned host copy
    std::vector<std::vector<unsigned>> rois;   // per output tensor: n x 4
    std::vector<std::vector<unsigned>> windows;   // per node: n x {x,y,w,h} source window (crop-type nodes)
    float* d_enc_boxes = nullptr;
    int* d_enc_labels = nullptr;
    int* d_matches = nullptr;         // box IoU matcher output [n][anchors]
    std::vector<float> boxes;        // metadata after the graph (normalized ltrb)
    std::vector<int> labels, counts;
    std::vector<int> file_labels;    // file source: class label per sample
    std::vector<std::string> names;  // file source: file name per sample
    size_t padded = 0;
    std::vector<int> source_wh;              // n x {width, height} of the whole source images (before a decoder crop)
    std::vector<unsigned> decoder_windows;   // fused JPEG crop / random bbox crop: n x {x,y,w,h} inside the whole images
    std::vector<float> bbox_crop_windows;    // random bbox crop: n x {x,y,w,h} as fractions of the image, as sampled
    unsigned decoder_batch_seed = 0;
    size_t n = 0;
    std::string error;
    std::vector<std::pair<const void*, std::vector<int>>> int_params;       // per-sample parameter values this batch
    std::vector<std::pair<const void*, std::vector<float>>> float_params;   // was built with, by parameter object
    std::vector<cudaEvent_t> step_ev;        // profiling: before the upload, after it, after every launch of the batch
    bool step_ev_valid = false;              // the events of this slot were recorded for the batch it holds
};

// One line of the per-launch device timing (profiling on): the name of the step, the device time it has taken so far
// and the number of batches measured.
struct StepTiming {
    std::string name;
    double gpu_us = 0.0;
    unsigned long long batches = 0;
};

// RB200_LOG_LEVEL: 0 = silent, 1 = errors (default), 2 = also the plan at verify and a timing summary at release.
int log_level();

class Pipeline {
   public:
    Pipeline(size_t batch, int gpu_id, size_t prefetch_depth, RocalTensorOutputType out_dtype);
    ~Pipeline();

    // ---- graph building (user thread, before verify) ----
    TensorImpl* add_source(unsigned max_w, unsigned max_h, bool is_output);
    TensorImpl* add_file_source(const std::string& root, unsigned shard_id, unsigned shard_count, bool shuffle, bool loop,
                                unsigned max_w, unsigned max_h, bool is_output, int last_batch_policy, bool pad_last_batch_repeated);
    TensorImpl* add_coco_source(const std::string& root, const std::string& json_path, bool avoid_class_remapping, unsigned shard_id,
                                unsigned shard_count, bool shuffle, bool loop, unsigned max_w, unsigned max_h, bool is_output,
                                int last_batch_policy, bool pad_last_batch_repeated);
    // rocalFusedJpegCrop*: every image of an encoded source is cut to a random-resized-crop window before the graph
    // Per-launch device timing with CUDA events (off by default; RB200_PROFILE=1 in the environment turns it on for
    // every context). Must be chosen before verify().
    // The per-sample values of a parameter for the batch that run() returned (0 values when it has none).
    size_t batch_int_array(const void* core, int* out, size_t n);
    size_t batch_float_array(const void* core, float* out, size_t n);
    void set_profiling(bool on);
    std::vector<StepTiming> step_timing();
    void set_random_crop_decoder(const RandomCropRanges& r);
    // rocalRandomBBoxCrop: every image (and its boxes) of the source is cut to a window sampled around the boxes
    void set_random_bbox_crop(bool all_boxes_overlap, bool has_shape, uint32_t seed);
    void bbox_crop_windows(float* xywh);
    void decoder_crop_windows(unsigned* xywh, unsigned* batch_seed);
    void reset_loaders();
    // Orders the reuse of the held batch's buffers behind the work already queued on `consumer_stream`
    void consumer_fence(void* consumer_stream);
    void set_arithmetic(int mode);
    void set_wait_probe(unsigned long long wait_cycles, int skip_row);
    void image_labels(int* buf);
    TensorListImpl* image_label_list();   // rocalGetImageLabels: one int32 host tensor per sample, buffers consecutive
    void image_ids(int* buf);
    const std::vector<std::string>& image_names();
    size_t last_batch_padded_size();
    void source_sizes(int* wh);
    void roi_image_sizes(int* wh);
    TensorImpl* add_node(Node node, TensorImpl* in, unsigned out_w, unsigned out_h, RocalTensorLayout lay,
                         RocalTensorOutputType dt, bool is_output, TensorImpl* in2 = nullptr);
    void set_box_encoder(const float* anchors, size_t num_anchors, float criteria, const float* means,
                         const float* stds, bool offset, float scale);
    void set_box_matcher(const float* anchors, size_t num_anchors, float high, float low, bool allow_low_quality);
    // The user sees the outputs in the order in which they were declared (MasterGraph::set_output, master_graph.cpp:337-349).
    void mark_output(TensorImpl* t);
    void verify();

    // ---- feeding (user thread) ----
    void feed(InputBatch&& b);
    void stage_boxes(const float* ltrb, const int* labels, const int* counts, size_t n);
    void stage_anchors(TensorImpl* t, const float* ax, const float* ay, size_t n);
    void stage_affine(TensorImpl* t, const float* m6, size_t n);

    // ---- running ----
    void run();
    size_t remaining();

    // ---- access ----
    int batch() const { return (int)_batch; }
    int gpu_id() const { return _gpu_id; }
    cudaStream_t stream() const { return _stream; }
    TensorListImpl* outputs() { return &_output_list; }
    TensorImpl* tensor(int id) { return _tensors[id].get(); }
    bool owns(const void* t) const;
    MetaListImpl* encoded_meta();
    void encoded(float** boxes, int** labels, size_t* num_anchors);
    void copy_encoded(float* boxes, int* labels);
    TensorListImpl* matched_indices();
    // rocalGetBoundingBoxCount / Cords / Label: per-sample host tensors over the held slot's boxes
    unsigned bounding_box_count();
    TensorListImpl* bounding_box_cords();
    TensorListImpl* bounding_box_labels();
    void matches(int** dev, size_t* num_anchors);
    void current_boxes(std::vector<float>& ltrb, std::vector<int>& labels, std::vector<int>& counts);
    void crop_windows(TensorImpl* t, unsigned* xywh);
    void to_tensor(void* out_ptr, int layout, int dtype, const float* mul, const float* add, bool reverse, int mem_type);
    TimingInfo timing();
    unsigned long long h2d_bytes() const { return _h2d_bytes.load(); }
    void set_upload_mode(int mode) { _upload_mode = mode; }
    RocalTensorOutputType default_dtype() const { return _out_dtype; }

    // ---- error capture (Context::capture_error, include/pipeline/context.h:41-51) ----
    void capture_error(const std::string& msg);
    RocalStatus status();
    const char* error_message();
    bool verified() const { return _verified; }

    void sync_copy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind);

   private:
    void worker_loop();
    void top_up();
    void process(InputBatch& b, Slot& s, int slot_idx);
    void update_nodes(const InputBatch& b, Slot& s);
    void ensure_arena(int which, size_t bytes);
    bool source_footprint(const uint8_t* h_tab, size_t i, int W, int H, int& x0, int& y0, int& x1, int& y1) const;
    void upload_sources(InputBatch& b, int a, const uint8_t* h_tab);
    void plan();
    void ssd_crop(Node& nd, const std::vector<int>& in_w, const std::vector<int>& in_h, Slot& s);
    void transform_boxes_window(Slot& s, const std::vector<unsigned>& x1, const std::vector<unsigned>& y1,
                                const std::vector<unsigned>& cw, const std::vector<unsigned>& ch,
                                const std::vector<int>& in_w, const std::vector<int>& in_h, bool by_centre);
    void mirror_boxes(Slot& s, const std::vector<int>& flags, bool vertical = false);
    void rotate_boxes(Slot& s, const std::vector<float>& angle_deg, const std::vector<int>& in_w, const std::vector<int>& in_h,
                      int dst_w, int dst_h);

    size_t _batch;
    int _gpu_id;
    size_t _depth;
    RocalTensorOutputType _out_dtype;
    cudaStream_t _stream = nullptr;
    // Box upload, encoder and matcher run on their own stream, beside the pixel kernels of the same batch; the batch's
    // completion event waits for both.
    cudaStream_t _meta_stream = nullptr;
    cudaEvent_t _meta_done = nullptr, _box_stage_free = nullptr;
    bool _verified = false;

    std::vector<std::unique_ptr<TensorImpl>> _tensors;
    std::vector<Node> _nodes;
    std::vector<Step> _steps;
    TensorListImpl _output_list;
    std::vector<int> _output_order;   // tensor ids in the order they became outputs (creation with is_output, rocalSetOutputs)
    int _source = -1;

    // box encoder
    bool _box_encoder = false;
    std::vector<float> _anchors;
    float* _d_anchors = nullptr;
    rb200_box_encoder_params _enc{};
    float* _d_boxes = nullptr;
    int *_d_labels = nullptr, *_d_offsets = nullptr;
    void* _h_box_stage = nullptr;
    size_t _box_capacity = 0;
    std::unique_ptr<TensorImpl> _enc_boxes_t, _enc_labels_t;   // views handed out by rocalGetEncodedBoxesAndLables
    TensorListImpl _enc_list_boxes, _enc_list_labels;
    MetaListImpl _enc_meta;

    // per-sample views of the current batch's boxes (rebuilt by rocalRun)
    std::vector<std::unique_ptr<TensorImpl>> _bbox_t, _bbox_label_t;
    TensorListImpl _bbox_list, _bbox_label_list;
    std::vector<std::unique_ptr<TensorImpl>> _label_t;
    std::vector<int> _label_values;
    TensorListImpl _label_list;
    void refresh_box_views();

    // box IoU matcher
    bool _box_matcher = false;
    std::vector<float> _match_anchors;
    float* _d_match_anchors = nullptr;
    rb200_box_matcher_params _match{};
    std::unique_ptr<TensorImpl> _matches_t;
    TensorListImpl _match_list;

    // staging for extensions (attached to the next fed batch)
    InputBatch _staged;

    // rocalCreateCOCOReader only records its arguments; rocalJpegCOCOFileSource builds the reader
    std::string _coco_json;
    bool _coco_avoid_remap = false;
    std::string _file_list;
    bool _coco_source = false;
   public:
    void note_coco_reader(const std::string& json, bool avoid_remap) { _coco_json = json; _coco_avoid_remap = avoid_remap; }
    // rocalCreateLabelReader with a file list / rocalCreateTextFileBasedLabelReader: the next folder source reads this list
    void note_file_list(const std::string& list_path) { _file_list = list_path; }
    const std::string& coco_json() const { return _coco_json; }
    bool coco_avoid_remap() const { return _coco_avoid_remap; }
   private:
    // folder reader (rocalJpegFileSource): batches are fed by the pipeline itself
    std::unique_ptr<FileSource> _files;

    // JPEG front-end (created when the first encoded batch arrives)
    JpegDecoder _jpeg;
    std::vector<unsigned char*> _jpeg_dst;
    std::vector<int> _decode_h;                            // decoded height of each image
    std::vector<size_t> _decode_off;                       // arena offset of each decoded image (the view may start inside it)
    std::unique_ptr<RandomCropWindowSampler> _crop_dec;    // fused JPEG crop source
    std::vector<size_t> _jpeg_pitch;

    // input arenas (double buffered)
    void* _arena[2] = {nullptr, nullptr};
    size_t _arena_cap[2] = {0, 0};
    cudaEvent_t _arena_free[2] = {nullptr, nullptr};
    int _arena_next = 0;
    const uint8_t* _src_base = nullptr;
    std::vector<SampleView> _src_views;

    // ring
    std::vector<Slot> _slots;
    size_t _write = 0, _read = 0;
    int _held = -1;
    std::deque<InputBatch> _queue;
    size_t _in_flight = 0;
    std::mutex _m;
    std::condition_variable _cv_work, _cv_ready;
    std::thread _worker;
    bool _stop = false;

    // status
    std::mutex _err_m;
    std::string _error;
    RocalStatus _status = ROCAL_OK;

    // timing (us)
    std::atomic<unsigned long long> _t_load{0}, _t_decode{0}, _t_process{0}, _t_transfer{0};
    bool _profiling = false;
    std::mutex _prof_m;
    std::vector<StepTiming> _step_timing;    // [0] = upload, [1 + k] = step k, last = box encoder / matcher
    void collect_step_timing(Slot& s);
    std::string step_name(const Step& st) const;
    std::atomic<unsigned long long> _h2d_bytes{0};   // bytes the worker uploaded (pixels, tables, boxes)
    int _upload_mode = UPLOAD_ZERO_COPY;
    std::unique_ptr<BBoxCropSampler> _bbox_crop;
    std::vector<int> _whole_w, _whole_h;                  // the images the source views were cut from
    void* _norm_scratch = nullptr;                        // statistics scratch shared by the Normalize steps
    size_t _norm_scratch_bytes = 0;
    int _arith = RB200_ARITH_EXACT;                       // arithmetic of the colour operators (rb200_set_arithmetic)
    std::atomic<unsigned long long> _probe_wait_cycles{0};  // self-test: non-zero = launch through the probe entries
    std::atomic<int> _probe_skip_row{-1};
};

#define RB200_THROW(msg) throw std::runtime_error(std::string(msg))
#define RB200_CUDA(call)                                                                              \
    do {                                                                                              \
        cudaError_t _e = (call);                                                                      \
        if (_e != cudaSuccess)                                                                        \
            throw std::runtime_error(std::string(#call) + ": " + cudaGetErrorString(_e));             \
    } while (0)

}  // namespace rb200
