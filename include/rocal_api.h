/*
 * rocal_api.h — the subset of the rocAL C API that the B200 augmentation path implements,
 * with the reference's names, argument order, defaults and error behaviour, so that code
 * written against rocAL's headers for these calls compiles and links against
 * librocal_b200.so unchanged.
 *
 * Like the reference, these are C++ signatures with C linkage (they take std::vector and
 * default arguments). The C-callable twin of every entry point is declared in rb200.h.
 *
 * Each declaration names the reference declaration it stands in for
 * (paths relative to the reference's rocAL/include/api/).
 *
 * Behaviour shared by all calls (rocal_api.h:42-62 of the reference): a null context or input
 * returns nullptr / ROCAL_CONTEXT_INVALID; any failure inside a call is caught, stored in the
 * context (rocalGetStatus / rocalGetErrorMessage) and printed to stderr; tensor-returning
 * calls then return nullptr.
 */
#ifndef ROCAL_B200_ROCAL_API_H
#define ROCAL_B200_ROCAL_API_H

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#ifndef ROCAL_API_CALL
#define ROCAL_API_CALL
#endif
#ifndef ROCAL_B200_EXPORT
#define ROCAL_B200_EXPORT __attribute__((visibility("default")))
#endif

/* ---- handles and enums (rocal_api_types.h:61-63, 102-527) ---- */
typedef void* RocalFloatParam;
typedef void* RocalIntParam;
typedef void* RocalContext;

struct TimingInfo {
    long long unsigned load_time;
    long long unsigned decode_time;
    long long unsigned process_time;
    long long unsigned transfer_time;
};

struct ROIxywh {
    unsigned x, y, w, h;
};

enum RocalStatus {
    ROCAL_OK = 0,
    ROCAL_CONTEXT_INVALID,
    ROCAL_RUNTIME_ERROR,
    ROCAL_UPDATE_PARAMETER_FAILED,
    ROCAL_INVALID_PARAMETER_TYPE
};
enum RocalImageColor { ROCAL_COLOR_RGB24 = 0, ROCAL_COLOR_BGR24 = 1, ROCAL_COLOR_U8 = 2, ROCAL_COLOR_RGB_PLANAR = 3 };
enum RocalProcessMode { ROCAL_PROCESS_GPU = 0, ROCAL_PROCESS_CPU = 1 };
enum RocalImageSizeEvaluationPolicy {
    ROCAL_USE_MAX_SIZE = 0,
    ROCAL_USE_USER_GIVEN_SIZE = 1,
    ROCAL_USE_MOST_FREQUENT_SIZE = 2,
    ROCAL_USE_USER_GIVEN_SIZE_RESTRICTED = 3,
    ROCAL_USE_MAX_SIZE_RESTRICTED = 4
};
enum RocalTensorLayout {
    ROCAL_NHWC = 0, ROCAL_NCHW = 1, ROCAL_NFHWC = 2, ROCAL_NFCHW = 3, ROCAL_NHW = 4,
    ROCAL_NFT = 5, ROCAL_NTF = 6, ROCAL_NDHWC = 7, ROCAL_NCDHW = 8, ROCAL_NONE = 9
};
enum RocalTensorOutputType {
    ROCAL_FP32 = 0, ROCAL_FP16 = 1, ROCAL_UINT8 = 2, ROCAL_INT8 = 3, ROCAL_UINT32 = 4, ROCAL_INT32 = 5, ROCAL_INT16 = 6
};
enum RocalDecoderType {
    ROCAL_DECODER_TJPEG = 0, ROCAL_DECODER_OPENCV = 1, ROCAL_DECODER_VIDEO_FFMPEG_SW = 2,
    ROCAL_DECODER_AUDIO_GENERIC = 3, ROCAL_DECODER_VIDEO_ROCDECODE = 4, ROCAL_DECODER_ROCJPEG = 5
};
enum RocalOutputMemType { ROCAL_MEMCPY_HOST = 0, ROCAL_MEMCPY_GPU = 1, ROCAL_MEMCPY_PINNED = 2 };
enum RocalResizeScalingMode {
    ROCAL_SCALING_MODE_DEFAULT = 0, ROCAL_SCALING_MODE_STRETCH = 1, ROCAL_SCALING_MODE_NOT_SMALLER = 2,
    ROCAL_SCALING_MODE_NOT_LARGER = 3, ROCAL_SCALING_MODE_MIN_MAX = 4
};
enum RocalResizeInterpolationType {
    ROCAL_NEAREST_NEIGHBOR_INTERPOLATION = 0, ROCAL_LINEAR_INTERPOLATION = 1, ROCAL_CUBIC_INTERPOLATION = 2,
    ROCAL_LANCZOS_INTERPOLATION = 3, ROCAL_GAUSSIAN_INTERPOLATION = 4, ROCAL_TRIANGULAR_INTERPOLATION = 5
};
enum RocalTensorBackend { ROCAL_CPU = 0, ROCAL_GPU = 1 };
enum class RocalROICordsType { ROCAL_LTRB = 0, ROCAL_XYWH = 1 };
enum RocalExternalSourceMode {
    ROCAL_EXTSOURCE_FNAME = 0, ROCAL_EXTSOURCE_RAW_COMPRESSED = 1, ROCAL_EXTSOURCE_RAW_UNCOMPRESSED = 2
};
/* Types that only absent entry points take; kept so that sources naming them still compile (rocal_api_types.h:163-203,
 * 411-449, 500-509). */
enum RocalFlipAxis { ROCAL_FLIP_HORIZONTAL = 0, ROCAL_FLIP_VERTICAL = 1 };
enum RocalDecodeDevice { ROCAL_HW_DECODE = 0, ROCAL_SW_DECODE = 1 };
enum RocalAudioBorderType { ROCAL_ZERO = 0, ROCAL_CLAMP = 1, ROCAL_REFLECT = 2 };
enum RocalOutOfBoundsPolicy { ROCAL_PAD = 0, ROCAL_TRIMTOSHAPE = 1, ROCAL_ERROR = 2 };
enum RocalMelScaleFormula { ROCAL_MELSCALE_SLANEY = 0, ROCAL_MELSCALE_HTK = 1 };
enum RocalMissingComponentsBehaviour { ROCAL_MISSING_COMPONENT_ERROR = 0, ROCAL_MISSING_COMPONENT_SKIP = 1, ROCAL_MISSING_COMPONENT_EMPTY = 2 };
enum RocalLastBatchPolicy { ROCAL_LAST_BATCH_FILL = 0, ROCAL_LAST_BATCH_DROP = 1, ROCAL_LAST_BATCH_PARTIAL = 2 };
struct RocalShardingInfo {   /* rocal_api_types.h:470-495: the same members and the same two constructors */
    RocalLastBatchPolicy last_batch_policy = ROCAL_LAST_BATCH_FILL;
    bool pad_last_batch_repeated = false;
    bool stick_to_shard = true;
    int32_t shard_size = -1;
    RocalShardingInfo() = default;
    RocalShardingInfo(RocalLastBatchPolicy policy, bool pad_repeated, bool stick, int size)
        : last_batch_policy(policy), pad_last_batch_repeated(pad_repeated), stick_to_shard(stick), shard_size(size) {}
};

/* ---- tensors (rocal_api_tensor.h:38-94) ---- */
class rocalTensor {
   public:
    virtual ~rocalTensor() = default;
    virtual void* buffer() = 0;
    virtual unsigned copy_data(void* user_buffer, RocalOutputMemType external_mem_type = ROCAL_MEMCPY_HOST) = 0;
    virtual unsigned copy_data(void* user_buffer, unsigned x_offset, unsigned y_offset, unsigned max_cols, unsigned max_rows) = 0;
    virtual unsigned num_of_dims() = 0;
    virtual unsigned batch_size() = 0;
    virtual std::vector<size_t> dims() = 0;
    virtual std::vector<size_t> strides() = 0;
    virtual RocalTensorLayout layout() = 0;
    virtual RocalTensorBackend backend() = 0;
    virtual RocalTensorOutputType data_type() = 0;
    virtual RocalOutputMemType mem_type() = 0;
    virtual size_t data_size() = 0;
    virtual RocalROICordsType roi_type() = 0;
    virtual size_t get_roi_dims_size() = 0;
    virtual void copy_roi(void* roi_buffer) = 0;
    virtual std::vector<size_t> shape() = 0;
    virtual void set_dims(std::vector<size_t> dims) = 0;
    virtual void set_mem_handle(void* buffer) = 0;
    virtual void set_tensor_layout(RocalTensorLayout layout) = 0;
    virtual uint64_t data_type_size() = 0;
};
class rocalTensorList {
   public:
    virtual ~rocalTensorList() = default;
    virtual uint64_t size() = 0;
    virtual rocalTensor* at(size_t index) = 0;
};
class rocalListOfTensorList {
   public:
    virtual ~rocalListOfTensorList() = default;
    virtual uint64_t size() = 0;
    virtual rocalTensorList* at(size_t index) = 0;
};
typedef rocalTensor* RocalTensor;
typedef rocalTensorList* RocalTensorList;
typedef rocalListOfTensorList* RocalMetaData;

#define RB200_ROCAL extern "C" ROCAL_B200_EXPORT

/* ---- life cycle (rocal_api.h:83-110) ---- */
RB200_ROCAL RocalContext ROCAL_API_CALL rocalCreate(size_t batch_size, RocalProcessMode affinity, int gpu_id = 0,
                                                     size_t cpu_thread_count = 1, size_t prefetch_queue_depth = 3,
                                                     RocalTensorOutputType output_tensor_data_type = ROCAL_FP32);
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalVerify(RocalContext context);
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalRun(RocalContext context);
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalRelease(RocalContext rocal_context);

/* ---- parameters (rocal_api_parameters.h:39-161) ---- */
RB200_ROCAL void ROCAL_API_CALL rocalSetSeed(unsigned seed);
RB200_ROCAL unsigned ROCAL_API_CALL rocalGetSeed();
RB200_ROCAL RocalIntParam ROCAL_API_CALL rocalCreateIntUniformRand(int start, int end);
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalUpdateIntUniformRand(int start, int end, RocalIntParam updating_obj);
RB200_ROCAL int ROCAL_API_CALL rocalGetIntValue(RocalIntParam obj);
RB200_ROCAL float ROCAL_API_CALL rocalGetFloatValue(RocalFloatParam obj);
RB200_ROCAL RocalFloatParam ROCAL_API_CALL rocalCreateFloatUniformRand(float start, float end);
RB200_ROCAL RocalFloatParam ROCAL_API_CALL rocalCreateFloatParameter(float val);
RB200_ROCAL RocalIntParam ROCAL_API_CALL rocalCreateIntParameter(int val);
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalUpdateFloatParameter(float new_val, RocalFloatParam input_obj);
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalUpdateIntParameter(int new_val, RocalIntParam input_obj);
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalUpdateFloatUniformRand(float start, float end, RocalFloatParam updating_obj);
RB200_ROCAL RocalIntParam ROCAL_API_CALL rocalCreateIntRand(const int* values, const double* frequencies, unsigned size);
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalUpdateIntRand(const int* values, const double* frequencies, unsigned size, RocalIntParam updating_obj);
RB200_ROCAL RocalFloatParam ROCAL_API_CALL rocalCreateFloatRand(const float* values, const double* frequencies, unsigned size);
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalUpdateFloatRand(const float* values, const double* frequencies, unsigned size, RocalFloatParam updating_obj);

/* ---- input: the external source (rocal_api_data_loaders.h:961-970, rocal_api_data_transfer.h:101-105) in its
 * three modes. ROCAL_EXTSOURCE_RAW_UNCOMPRESSED: each fed buffer is a max_height x max_width x channels slot with
 * the valid roi.w x roi.h region at its origin (image_read_and_decode.cpp:217-244 of the reference).
 * ROCAL_EXTSOURCE_RAW_COMPRESSED: each buffer is a JPEG stream whose length is roi.h. ROCAL_EXTSOURCE_FNAME: the
 * names in input_images_names are JPEG files. JPEG input is decoded on the GPU (nvJPEG). ---- */
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalJpegExternalFileSource(
    RocalContext p_context, RocalImageColor rocal_color_format, bool is_output = false, bool shuffle = false,
    bool loop = false, RocalImageSizeEvaluationPolicy decode_size_policy = ROCAL_USE_MOST_FREQUENT_SIZE,
    unsigned max_width = 0, unsigned max_height = 0, RocalDecoderType rocal_decoder_type = ROCAL_DECODER_TJPEG,
    RocalExternalSourceMode external_source_mode = ROCAL_EXTSOURCE_FNAME,
    RocalShardingInfo rocal_sharding_info = RocalShardingInfo());
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalExternalSourceFeedInput(
    RocalContext p_context, const std::vector<std::string>& input_images_names, bool is_labels,
    const std::vector<unsigned char*>& input_buffer, const std::vector<ROIxywh>& roi_xywh, unsigned int max_width,
    unsigned int max_height, unsigned int channels, RocalExternalSourceMode mode, RocalTensorLayout layout, bool eos);

/* ---- input: JPEG files in a folder tree (rocal_api_data_loaders.h:51-90) with the folder label reader
 * (rocal_api_meta_data.h:43,153-171) and the loader controls (rocal_api_data_loaders.h: rocalResetLoaders;
 * rocal_api_info.h: rocalGetLastBatchPaddedSize). internal_shard_count must be 1: one context drives one GPU.
 * max_width / max_height bound the decoded size and must be given. ---- */
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalJpegFileSource(
    RocalContext context, const char* source_path, RocalImageColor rocal_color_format, unsigned internal_shard_count,
    bool is_output, bool shuffle = false, bool loop = false,
    RocalImageSizeEvaluationPolicy decode_size_policy = ROCAL_USE_MOST_FREQUENT_SIZE, unsigned max_width = 0,
    unsigned max_height = 0, RocalDecoderType rocal_decoder_type = ROCAL_DECODER_TJPEG,
    RocalShardingInfo rocal_sharding_info = RocalShardingInfo());
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalJpegFileSourceSingleShard(
    RocalContext context, const char* source_path, RocalImageColor rocal_color_format, unsigned shard_id,
    unsigned shard_count, bool is_output, bool shuffle = false, bool loop = false,
    RocalImageSizeEvaluationPolicy decode_size_policy = ROCAL_USE_MOST_FREQUENT_SIZE, unsigned max_width = 0,
    unsigned max_height = 0, RocalDecoderType rocal_decoder_type = ROCAL_DECODER_TJPEG,
    RocalShardingInfo rocal_sharding_info = RocalShardingInfo());
/* rocal_api_data_loaders.h:462-506: the folder source with a random-resized-crop window per image
 * (area_factor = {min, max} fraction of the image area, aspect_ratio = {min, max} width / height). */
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalFusedJpegCrop(
    RocalContext context, const char* source_path, RocalImageColor rocal_color_format, unsigned num_threads, bool is_output,
    std::vector<float>& area_factor, std::vector<float>& aspect_ratio, unsigned num_attempts, bool shuffle = false,
    bool loop = false, RocalImageSizeEvaluationPolicy decode_size_policy = ROCAL_USE_MOST_FREQUENT_SIZE, unsigned max_width = 0,
    unsigned max_height = 0, RocalShardingInfo rocal_sharding_info = RocalShardingInfo());
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalFusedJpegCropSingleShard(
    RocalContext context, const char* source_path, RocalImageColor color_format, unsigned shard_id, unsigned shard_count,
    bool is_output, std::vector<float>& area_factor, std::vector<float>& aspect_ratio, unsigned num_attempts,
    bool shuffle = false, bool loop = false, RocalImageSizeEvaluationPolicy decode_size_policy = ROCAL_USE_MOST_FREQUENT_SIZE,
    unsigned max_width = 0, unsigned max_height = 0, RocalShardingInfo rocal_sharding_info = RocalShardingInfo());
/* COCO detection datasets (rocal_api_meta_data.h:89, rocal_api_data_loaders.h:163-174,257-269): boxes and labels come
 * from the annotation file and follow the graph's crops and mirrors. */
RB200_ROCAL RocalMetaData ROCAL_API_CALL rocalCreateCOCOReader(RocalContext rocal_context, const char* source_path, bool is_output,
                                                             bool mask = false, bool ltrb = true, bool is_box_encoder = false,
                                                             bool avoid_class_remapping = false, bool aspect_ratio_grouping = false,
                                                             bool is_box_iou_matcher = false);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalJpegCOCOFileSource(
    RocalContext context, const char* source_path, const char* json_path, RocalImageColor color_format, unsigned internal_shard_count,
    bool is_output, bool shuffle = false, bool loop = false,
    RocalImageSizeEvaluationPolicy decode_size_policy = ROCAL_USE_MOST_FREQUENT_SIZE, unsigned max_width = 0, unsigned max_height = 0,
    RocalDecoderType rocal_decoder_type = ROCAL_DECODER_TJPEG, RocalShardingInfo rocal_sharding_info = RocalShardingInfo());
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalJpegCOCOFileSourceSingleShard(
    RocalContext context, const char* source_path, const char* json_path, RocalImageColor color_format, unsigned shard_id,
    unsigned shard_count, bool is_output, bool shuffle = false, bool loop = false,
    RocalImageSizeEvaluationPolicy decode_size_policy = ROCAL_USE_MOST_FREQUENT_SIZE, unsigned max_width = 0, unsigned max_height = 0,
    RocalDecoderType rocal_decoder_type = ROCAL_DECODER_TJPEG, RocalShardingInfo rocal_sharding_info = RocalShardingInfo());
/* rocal_api_data_loaders.h:193-239: the COCO source behind the random-crop decoder; the window cuts the pixels, the
 * boxes stay those of the whole image (only rocalRandomBBoxCrop, which is not built, moves boxes with a decode window). */
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalJpegCOCOFileSourcePartial(
    RocalContext p_context, const char* source_path, const char* json_path, RocalImageColor rocal_color_format,
    unsigned internal_shard_count, bool is_output, std::vector<float>& area_factor, std::vector<float>& aspect_ratio,
    unsigned num_attempts, bool shuffle = false, bool loop = false,
    RocalImageSizeEvaluationPolicy decode_size_policy = ROCAL_USE_MOST_FREQUENT_SIZE, unsigned max_width = 0,
    unsigned max_height = 0, RocalShardingInfo rocal_sharding_info = RocalShardingInfo());
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalJpegCOCOFileSourcePartialSingleShard(
    RocalContext p_context, const char* source_path, const char* json_path, RocalImageColor rocal_color_format,
    unsigned shard_id, unsigned shard_count, bool is_output, std::vector<float>& area_factor, std::vector<float>& aspect_ratio,
    unsigned num_attempts, bool shuffle = false, bool loop = false,
    RocalImageSizeEvaluationPolicy decode_size_policy = ROCAL_USE_MOST_FREQUENT_SIZE, unsigned max_width = 0,
    unsigned max_height = 0, RocalShardingInfo rocal_sharding_info = RocalShardingInfo());
RB200_ROCAL RocalMetaData ROCAL_API_CALL rocalCreateLabelReader(RocalContext rocal_context, const char* source_path,
                                                              const char* file_list_path = "");
/* rocal_api_meta_data.h:108: labels from a text file of "file_name label" lines; the following rocalJpegFileSource* reads
 * the listed files (relative to its source_path) in the list's order. */
RB200_ROCAL RocalMetaData ROCAL_API_CALL rocalCreateTextFileBasedLabelReader(RocalContext rocal_context, const char* source_path);
/* rocal_api_meta_data.h:171: one one-element int32 host tensor per sample; the buffers are consecutive, so
 * at(0)->buffer() reads as int[batch] (rb200_get_image_labels copies into a caller's array instead). */
RB200_ROCAL RocalTensorList ROCAL_API_CALL rocalGetImageLabels(RocalContext rocal_context);
RB200_ROCAL void ROCAL_API_CALL rocalGetOneHotImageLabels(RocalContext rocal_context, void* buf, int numOfClasses,
                                                         RocalOutputMemType output_mem_type);
RB200_ROCAL void ROCAL_API_CALL rocalGetImageSizes(RocalContext rocal_context, int* buf);
RB200_ROCAL void ROCAL_API_CALL rocalGetROIImageSizes(RocalContext rocal_context, int* buf);
RB200_ROCAL void ROCAL_API_CALL rocalGetImageId(RocalContext rocal_context, int* buf);
RB200_ROCAL unsigned ROCAL_API_CALL rocalGetImageNameLen(RocalContext rocal_context, int* buf);
RB200_ROCAL void ROCAL_API_CALL rocalGetImageName(RocalContext rocal_context, char* buf);
RB200_ROCAL void ROCAL_API_CALL rocalResetLoaders(RocalContext context);
RB200_ROCAL size_t ROCAL_API_CALL rocalGetLastBatchPaddedSize(RocalContext rocal_context);

/* ---- augmentations (rocal_api_augmentation.h; line of each reference declaration in brackets) ---- */
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalResize /* [67] */ (
    RocalContext context, RocalTensor input, unsigned dest_width, unsigned dest_height, bool is_output,
    RocalResizeScalingMode scaling_mode = ROCAL_SCALING_MODE_STRETCH, std::vector<unsigned> max_size = {},
    unsigned resize_shorter = 0, unsigned resize_longer = 0,
    RocalResizeInterpolationType interpolation_type = ROCAL_LINEAR_INTERPOLATION,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalResizeMirrorNormalize /* [98] */ (
    RocalContext p_context, RocalTensor p_input, unsigned dest_width, unsigned dest_height, std::vector<float>& mean,
    std::vector<float>& std_dev, bool is_output, RocalResizeScalingMode scaling_mode = ROCAL_SCALING_MODE_STRETCH,
    std::vector<unsigned> max_size = {}, unsigned resize_shorter = 0, unsigned resize_longer = 0,
    RocalResizeInterpolationType interpolation_type = ROCAL_LINEAR_INTERPOLATION, RocalIntParam mirror = NULL,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalRotate /* [200] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalFloatParam angle = NULL, unsigned dest_width = 0,
    unsigned dest_height = 0, RocalResizeInterpolationType interpolation_type = ROCAL_LINEAR_INTERPOLATION,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalRotateFixed /* [220] */ (
    RocalContext context, RocalTensor input, float angle, bool is_output, unsigned dest_width = 0,
    unsigned dest_height = 0, RocalResizeInterpolationType interpolation_type = ROCAL_LINEAR_INTERPOLATION,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalBrightness /* [237] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalFloatParam alpha = NULL, RocalFloatParam beta = NULL,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalBrightnessFixed /* [253] */ (
    RocalContext context, RocalTensor input, float alpha, float beta, bool is_output,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalContrast /* [302] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalFloatParam contrast_factor = NULL,
    RocalFloatParam contrast_center = NULL, RocalTensorLayout output_layout = ROCAL_NONE,
    RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalContrastFixed /* [319] */ (
    RocalContext context, RocalTensor input, float contrast_factor, float contrast_center, bool is_output,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalFlip /* [336] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalIntParam horizonal_flag = NULL,
    RocalIntParam vertical_flag = NULL, RocalTensorLayout output_layout = ROCAL_NONE,
    RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalFlipFixed /* [352] */ (
    RocalContext context, RocalTensor input, int horizonal_flag, int vertical_flag, bool is_output,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalWarpAffine /* [422] */ (
    RocalContext context, RocalTensor input, bool is_output, unsigned dest_height = 0, unsigned dest_width = 0,
    RocalFloatParam x0 = NULL, RocalFloatParam x1 = NULL, RocalFloatParam y0 = NULL, RocalFloatParam y1 = NULL,
    RocalFloatParam o0 = NULL, RocalFloatParam o1 = NULL,
    RocalResizeInterpolationType interpolation_type = ROCAL_LINEAR_INTERPOLATION,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalWarpAffineFixed /* [449] */ (
    RocalContext context, RocalTensor input, float x0, float x1, float y0, float y1, float o0, float o1,
    bool is_output, unsigned int dest_height = 0, unsigned int dest_width = 0,
    RocalResizeInterpolationType interpolation_type = ROCAL_LINEAR_INTERPOLATION,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalBlend /* [382] */ (
    RocalContext context, RocalTensor input1, RocalTensor input2, bool is_output, RocalFloatParam ratio = NULL,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalBlendFixed /* [399] */ (
    RocalContext context, RocalTensor input1, RocalTensor input2, float ratio, bool is_output,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalGamma /* [269] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalFloatParam gamma = NULL,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalGammaFixed /* [285] */ (
    RocalContext context, RocalTensor input, float gamma, bool is_output, RocalTensorLayout output_layout = ROCAL_NONE,
    RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalColorTemp /* [667] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalIntParam adjustment = NULL,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalColorTempFixed /* [683] */ (
    RocalContext context, RocalTensor input, int adjustment, bool is_output, RocalTensorLayout output_layout = ROCAL_NONE,
    RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalExposure /* [763] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalFloatParam exposure_factor = NULL,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalExposureFixed /* [779] */ (
    RocalContext context, RocalTensor input, float exposure_factor, bool is_output, RocalTensorLayout output_layout = ROCAL_NONE,
    RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalHue /* [794] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalFloatParam hue = NULL,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalHueFixed /* [810] */ (
    RocalContext context, RocalTensor input, float hue, bool is_output, RocalTensorLayout output_layout = ROCAL_NONE,
    RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalSaturation /* [826] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalFloatParam saturation = NULL,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalSaturationFixed /* [842] */ (
    RocalContext context, RocalTensor input, float saturation, bool is_output,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalNormalize /* [1294] */ (
    RocalContext context, RocalTensor input, std::vector<unsigned>& axes, std::vector<float>& mean,
    std::vector<float>& std_dev, bool is_output, float scale = 1.0, float shift = 0.0,
    RocalTensorOutputType output_datatype = ROCAL_FP32);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalTranspose /* [1338] */ (
    RocalContext context, RocalTensor input, std::vector<unsigned> perm, bool is_output,
    RocalTensorLayout output_layout = ROCAL_NONE);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalColorTwist /* [878] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalFloatParam alpha = NULL, RocalFloatParam beta = NULL,
    RocalFloatParam hue = NULL, RocalFloatParam sat = NULL, RocalTensorLayout output_layout = ROCAL_NONE,
    RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalColorTwistFixed /* [900] */ (
    RocalContext context, RocalTensor input, float alpha, float beta, float hue, float sat, bool is_output,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalCropMirrorNormalize /* [925] */ (
    RocalContext context, RocalTensor input, unsigned crop_height, unsigned crop_width, float start_x, float start_y,
    std::vector<float>& mean, std::vector<float>& std_dev, bool is_output, RocalIntParam mirror = NULL,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalCrop /* [952] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalFloatParam crop_width = NULL,
    RocalFloatParam crop_height = NULL, RocalFloatParam crop_depth = NULL, RocalFloatParam crop_pox_x = NULL,
    RocalFloatParam crop_pos_y = NULL, RocalFloatParam crop_pos_z = NULL, RocalTensorLayout output_layout = ROCAL_NONE,
    RocalTensorOutputType output_datatype = ROCAL_UINT8);
/* The input unchanged, in the operator's own output tensor (same layout and type as the input). */
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalCopy /* [854] */ (RocalContext context, RocalTensor input, bool is_output);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalNop /* [863] */ (RocalContext context, RocalTensor input, bool is_output);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalCropResize /* [125] */ (
    RocalContext context, RocalTensor input, unsigned dest_width, unsigned dest_height, bool is_output, RocalFloatParam area = NULL,
    RocalFloatParam aspect_ratio = NULL, RocalFloatParam x_center_drift = NULL, RocalFloatParam y_center_drift = NULL,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalCropResizeFixed /* [151] */ (
    RocalContext context, RocalTensor input, unsigned dest_width, unsigned dest_height, bool is_output, float area,
    float aspect_ratio, float x_center_drift, float y_center_drift, RocalTensorLayout output_layout = ROCAL_NONE,
    RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalROIResize /* [175] */ (
    RocalContext context, RocalTensor input, unsigned dest_width, unsigned dest_height, bool is_output, unsigned roi_h,
    unsigned roi_w, float roi_pos_x = 0.0f, float roi_pos_y = 0.0f,
    RocalResizeInterpolationType interpolation_type = ROCAL_LINEAR_INTERPOLATION, RocalTensorLayout output_layout = ROCAL_NONE,
    RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalRandomCrop /* [1066] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalFloatParam crop_area_factor = NULL,
    RocalFloatParam crop_aspect_ratio = NULL, RocalFloatParam crop_pos_x = NULL, RocalFloatParam crop_pos_y = NULL,
    int num_of_attempts = 20, RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalCropFixed /* [977] */ (
    RocalContext context, RocalTensor input, unsigned crop_width, unsigned crop_height, unsigned crop_depth,
    bool is_output, float crop_pox_x, float crop_pos_y, float crop_pos_z,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalCropCenterFixed /* [1000] */ (
    RocalContext context, RocalTensor input, unsigned crop_width, unsigned crop_height, unsigned crop_depth,
    bool is_output, RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalResizeCropMirrorFixed /* [1022] */ (
    RocalContext context, RocalTensor input, unsigned dest_width, unsigned dest_height, bool is_output,
    unsigned crop_h, unsigned crop_w, RocalIntParam mirror, RocalTensorLayout output_layout = ROCAL_NONE,
    RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalResizeCropMirror /* [1045] */ (
    RocalContext context, RocalTensor input, unsigned dest_width, unsigned dest_height, bool is_output,
    RocalFloatParam crop_height = NULL, RocalFloatParam crop_width = NULL, RocalIntParam mirror = NULL,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);
RB200_ROCAL RocalTensor ROCAL_API_CALL rocalSSDRandomCrop /* [1091] */ (
    RocalContext context, RocalTensor input, bool is_output, RocalFloatParam threshold = NULL,
    RocalFloatParam crop_area_factor = NULL, RocalFloatParam crop_aspect_ratio = NULL,
    RocalFloatParam crop_pos_x = NULL, RocalFloatParam crop_pos_y = NULL, int num_of_attempts = 20,
    RocalTensorLayout output_layout = ROCAL_NONE, RocalTensorOutputType output_datatype = ROCAL_UINT8);

/* ---- outputs (rocal_api_data_transfer.h:43-83) ---- */
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalCopyToOutput(RocalContext context, unsigned char* out_ptr, size_t out_size);
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalToTensor(RocalContext rocal_context, void* out_ptr,
                                                     RocalTensorLayout tensor_format, RocalTensorOutputType tensor_output_type,
                                                     float multiplier0, float multiplier1, float multiplier2, float offset0,
                                                     float offset1, float offset2, bool reverse_channels,
                                                     RocalOutputMemType output_mem_type, int max_roi_height = 0,
                                                     int max_roi_width = 0);
RB200_ROCAL void ROCAL_API_CALL rocalSetOutputs(RocalContext p_context, unsigned int num_of_outputs, std::vector<RocalTensor>& output_images);
RB200_ROCAL RocalTensorList ROCAL_API_CALL rocalGetOutputTensors(RocalContext p_context);

/* ---- random bounding-box crop of the source images (rocal_api_meta_data.h:245) ---- */
RB200_ROCAL void ROCAL_API_CALL rocalRandomBBoxCrop(RocalContext p_context, bool all_boxes_overlap, bool no_crop,
                                                    RocalFloatParam aspect_ratio = NULL, bool has_shape = false, int crop_width = 0,
                                                    int crop_height = 0, int num_attempts = 1, RocalFloatParam scaling = NULL,
                                                    int total_num_attempts = 0, int64_t seed = 0);

/* ---- SSD box encoder (rocal_api_meta_data.h:270-286) ---- */
RB200_ROCAL void ROCAL_API_CALL rocalBoxEncoder(RocalContext p_context, std::vector<float>& anchors, float criteria,
                                                std::vector<float>& means, std::vector<float>& stds,
                                                bool offset = false, float scale = 1.0);
RB200_ROCAL void ROCAL_API_CALL rocalCopyEncodedBoxesAndLables(RocalContext p_context, float* boxes_buf, int* labels_buf);
RB200_ROCAL RocalMetaData ROCAL_API_CALL rocalGetEncodedBoxesAndLables(RocalContext p_context, int num_encoded_boxes);

/* ---- boxes of the current batch after the graph's crops and mirrors (rocal_api_meta_data.h:173-211): total
 * count, and one host tensor per sample - [count][4] float32 normalized ltrb, [count] int32 labels.
 * DIFFERS FROM THE REFERENCE: coordinates are fractions of the image the boxes currently belong to (0..1), whatever
 * the source. The reference's COCO reader keeps PIXEL coordinates (coco_meta_data_reader.cpp:140-325) and its meta
 * nodes rescale them along the graph, so a caller that took pixels from rocalGetBoundingBoxCords multiplies by the
 * output width / height here. ---- */
RB200_ROCAL unsigned ROCAL_API_CALL rocalGetBoundingBoxCount(RocalContext rocal_context);
RB200_ROCAL RocalTensorList ROCAL_API_CALL rocalGetBoundingBoxCords(RocalContext rocal_context);
RB200_ROCAL RocalTensorList ROCAL_API_CALL rocalGetBoundingBoxLabel(RocalContext rocal_context);

/* ---- box IoU matcher (rocal_api_meta_data.h:302-318) ---- */
RB200_ROCAL void ROCAL_API_CALL rocalBoxIouMatcher(RocalContext p_context, std::vector<float>& anchors, float high_threshold,
                                                   float low_threshold, bool allow_low_quality_matches = true);
RB200_ROCAL RocalTensorList ROCAL_API_CALL rocalGetMatchedIndices(RocalContext p_context);

/* ---- info (rocal_api_info.h:41-114) ---- */
RB200_ROCAL int ROCAL_API_CALL rocalGetOutputWidth(RocalContext rocal_context);
RB200_ROCAL int ROCAL_API_CALL rocalGetOutputHeight(RocalContext rocal_context);
RB200_ROCAL int ROCAL_API_CALL rocalGetOutputColorFormat(RocalContext rocal_context);
RB200_ROCAL size_t ROCAL_API_CALL rocalGetRemainingImages(RocalContext rocal_context);
RB200_ROCAL size_t ROCAL_API_CALL rocalIsEmpty(RocalContext rocal_context);
RB200_ROCAL size_t ROCAL_API_CALL rocalGetAugmentationBranchCount(RocalContext rocal_context);
RB200_ROCAL RocalStatus ROCAL_API_CALL rocalGetStatus(RocalContext rocal_context);
RB200_ROCAL const char* ROCAL_API_CALL rocalGetErrorMessage(RocalContext rocal_context);
RB200_ROCAL TimingInfo ROCAL_API_CALL rocalGetTimingInfo(RocalContext rocal_context);

#endif /* ROCAL_B200_ROCAL_API_H */
