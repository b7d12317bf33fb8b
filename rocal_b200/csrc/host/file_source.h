// Folder reader of the JPEG file source: the file list, labels, shard and batch sequence of
// rocalJpegFileSourceSingleShard + rocalCreateLabelReader.
//
// Follows the reference's readers for the parts a training script can observe:
//   * traversal: entries of the root sorted by name; every sub-folder is one class, numbered in that order;
//     a root that holds image files directly is a single class 0; files inside a folder sorted by name;
//     only image extensions are taken (rocAL/source/meta_data/label_reader_folders.cpp:95-137,
//     rocAL/source/readers/image/file_source_reader.cpp);
//   * shard i of S owns files [floor(N*i/S), floor(N*(i+1)/S)) of that list
//     (rocAL/source/readers/image/image_reader.cpp:48-67);
//   * last batch: FILL pads it (with the shard's last sample when pad_last_batch_repeated, else with samples
//     from the start of the shard), DROP leaves it out, PARTIAL pads like FILL and reports how many samples of
//     the last batch are padding (rocAL/include/api/rocal_api_types.h:455-495).
// Shuffling is a seeded std::shuffle per epoch (the reference shuffles unseeded).
#pragma once
#include <cstddef>
#include <cstdint>
#include <random>
#include <string>
#include <vector>

namespace rb200 {

struct FileBatch {
    std::vector<std::string> paths;
    std::vector<std::string> names;   // file name without the folder, as rocalGetImageName reports it
    std::vector<int> labels;
    size_t padded = 0;                // samples at the end of the batch that repeat earlier ones
    // detection datasets: ground-truth boxes of the batch (normalized ltrb), their labels, boxes per sample
    bool has_boxes = false;
    std::vector<float> boxes;
    std::vector<int> box_labels, counts;
};

// One sample of a dataset: the file, its class label (classification) and its boxes (detection).
struct FileEntry {
    std::string path, name;
    int label = 0;
    std::vector<float> boxes;
    std::vector<int> box_labels;
};

// A file list (rocalCreateLabelReader with file_list_path / rocalCreateTextFileBasedLabelReader): one
// whitespace-separated "file_name label" pair per line, names relative to `root`, lines that do not parse are
// skipped, the order of the list is kept, the reported name is the part after the last slash
// (rocAL/source/meta_data/text_file_meta_data_reader.cpp:71-93). Throws when the list cannot be opened or names
// no JPEG file.
std::vector<FileEntry> read_file_list(const std::string& list_path, const std::string& root);

class FileSource {
   public:
    enum LastBatch { FILL = 0, DROP = 1, PARTIAL = 2 };

    // Scans `root`; throws std::runtime_error when it cannot be read or holds no image.
    FileSource(const std::string& root, size_t batch, unsigned shard_id, unsigned shard_count, bool shuffle, bool loop,
               int last_batch_policy, bool pad_last_batch_repeated, unsigned seed);
    // A prepared list (the COCO reader's images with their boxes), in the order given.
    FileSource(std::vector<FileEntry> entries, bool with_boxes, size_t batch, unsigned shard_id, unsigned shard_count, bool shuffle,
               bool loop, int last_batch_policy, bool pad_last_batch_repeated, unsigned seed);

    size_t dataset_size() const { return _all.size(); }
    size_t shard_size() const { return _end - _begin; }
    size_t batches_per_epoch() const;
    // Batches of the current epoch that next() has not handed out yet (never 0 when looping).
    size_t batches_left() const;
    bool next(FileBatch& out);
    void reset();                     // start the next epoch (rocalResetLoaders)
    size_t last_batch_padded_size() const { return _last_padded; }

   private:
    void init_shard(unsigned shard_id, unsigned shard_count);
    void begin_epoch();

    std::vector<FileEntry> _all;
    bool _with_boxes = false;
    std::vector<size_t> _order;       // indices into _all for the current epoch, shard only
    size_t _begin = 0, _end = 0;
    size_t _batch;
    bool _shuffle, _loop;
    int _policy;
    bool _pad_repeat;
    unsigned _seed;
    unsigned _epoch = 0;
    size_t _cursor = 0;               // batches handed out in this epoch
    size_t _last_padded = 0;
};

}  // namespace rb200
