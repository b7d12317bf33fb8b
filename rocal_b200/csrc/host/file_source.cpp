#include "file_source.h"

#include <dirent.h>
#include <sys/stat.h>

#include <algorithm>
#include <cctype>
#include <fstream>
#include <sstream>
#include <stdexcept>

namespace rb200 {

namespace {

bool is_dir(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}
bool is_file(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

// JPEG is what the decoder takes; the reference's list of image extensions is longer
// (label_reader_folders.cpp:118) but its other formats have no decoder here.
bool is_jpeg_name(const std::string& name) {
    auto dot = name.find_last_of('.');
    if (dot == std::string::npos) return false;
    std::string ext = name.substr(dot + 1);
    std::transform(ext.begin(), ext.end(), ext.begin(), [](unsigned char c) { return (char)std::tolower(c); });
    return ext == "jpg" || ext == "jpeg";
}

std::vector<std::string> sorted_entries(const std::string& dir) {
    DIR* d = opendir(dir.c_str());
    if (!d) throw std::runtime_error("ERROR: Failed opening the directory at " + dir);
    std::vector<std::string> names;
    while (dirent* e = readdir(d)) {
        std::string n(e->d_name);
        if (n == "." || n == "..") continue;
        names.push_back(n);
    }
    closedir(d);
    std::sort(names.begin(), names.end());
    return names;
}

FileEntry make_entry(const std::string& path, const std::string& name, int label) {
    FileEntry e;
    e.path = path;
    e.name = name;
    e.label = label;
    return e;
}

}  // namespace

std::vector<FileEntry> read_file_list(const std::string& list_path, const std::string& root) {
    std::ifstream in(list_path.c_str());
    if (!in.good()) throw std::runtime_error("Can't open the metadata file at " + list_path);
    std::vector<FileEntry> out;
    std::string line;
    while (std::getline(in, line)) {
        std::istringstream fields(line);
        std::string rel;
        int label = 0;
        if (!(fields >> rel >> label)) continue;
        if (!is_jpeg_name(rel)) continue;
        const auto slash = rel.find_last_of("\\/");
        const std::string name = slash == std::string::npos ? rel : rel.substr(slash + 1);
        out.push_back(make_entry(root.empty() ? rel : root + "/" + rel, name, label));
    }
    if (out.empty()) throw std::runtime_error("no JPEG files named in " + list_path);
    return out;
}

FileSource::FileSource(std::vector<FileEntry> entries, bool with_boxes, size_t batch, unsigned shard_id, unsigned shard_count,
                       bool shuffle, bool loop, int last_batch_policy, bool pad_last_batch_repeated, unsigned seed)
    : _all(std::move(entries)), _with_boxes(with_boxes), _batch(batch), _shuffle(shuffle), _loop(loop), _policy(last_batch_policy),
      _pad_repeat(pad_last_batch_repeated), _seed(seed) {
    if (batch == 0) throw std::runtime_error("batch size must be positive");
    if (_policy < FILL || _policy > PARTIAL) throw std::runtime_error("bad last batch policy");
    if (_all.empty()) throw std::runtime_error("the dataset holds no image");
    init_shard(shard_id, shard_count);
}

void FileSource::init_shard(unsigned shard_id, unsigned shard_count) {
    if (shard_count == 0 || shard_id >= shard_count) throw std::runtime_error("shard_id must be smaller than shard_count");
    const size_t N = _all.size();
    _begin = N * shard_id / shard_count;
    _end = N * (shard_id + 1) / shard_count;
    if (_end == _begin) throw std::runtime_error("shard " + std::to_string(shard_id) + " of " + std::to_string(shard_count) + " is empty");
    begin_epoch();
}

FileSource::FileSource(const std::string& root, size_t batch, unsigned shard_id, unsigned shard_count, bool shuffle, bool loop,
                       int last_batch_policy, bool pad_last_batch_repeated, unsigned seed)
    : _batch(batch), _shuffle(shuffle), _loop(loop), _policy(last_batch_policy), _pad_repeat(pad_last_batch_repeated), _seed(seed) {
    if (batch == 0) throw std::runtime_error("batch size must be positive");
    if (_policy < FILL || _policy > PARTIAL) throw std::runtime_error("bad last batch policy");
    int label = 0;
    bool flat_done = false;
    for (const std::string& n : sorted_entries(root)) {
        const std::string p = root + "/" + n;
        if (is_file(p)) {
            if (!is_jpeg_name(n)) continue;
            if (!flat_done) {   // a root that holds files is one class; its files are taken once, sorted
                for (const std::string& f : sorted_entries(root))
                    if (is_file(root + "/" + f) && is_jpeg_name(f)) _all.push_back(make_entry(root + "/" + f, f, 0));
                flat_done = true;
            }
            break;              // "assume directory has only files" (label_reader_folders.cpp:127)
        } else if (is_dir(p)) {
            for (const std::string& f : sorted_entries(p))
                if (is_file(p + "/" + f) && is_jpeg_name(f)) _all.push_back(make_entry(p + "/" + f, f, label));
            label++;
        }
    }
    if (_all.empty()) throw std::runtime_error("no JPEG files found under " + root);
    init_shard(shard_id, shard_count);
}

void FileSource::begin_epoch() {
    _order.resize(_end - _begin);
    for (size_t i = 0; i < _order.size(); i++) _order[i] = _begin + i;
    if (_shuffle) {
        std::mt19937 gen(_seed * 2654435761u + _epoch);
        std::shuffle(_order.begin(), _order.end(), gen);
    }
    _cursor = 0;
}

size_t FileSource::batches_per_epoch() const {
    const size_t n = _order.size();
    return _policy == DROP ? n / _batch : (n + _batch - 1) / _batch;
}

size_t FileSource::batches_left() const {
    const size_t per = batches_per_epoch();
    if (_loop) return per;
    return per - _cursor;
}

bool FileSource::next(FileBatch& out) {
    const size_t per = batches_per_epoch();
    if (per == 0) return false;
    if (_cursor >= per) {
        if (!_loop) return false;
        _epoch++;
        begin_epoch();
    }
    const size_t n = _order.size();
    const size_t first = _cursor * _batch;
    out.paths.clear();
    out.names.clear();
    out.labels.clear();
    out.padded = 0;
    out.has_boxes = _with_boxes;
    out.boxes.clear();
    out.box_labels.clear();
    out.counts.clear();
    for (size_t k = 0; k < _batch; k++) {
        size_t pos = first + k;
        if (pos >= n) {
            pos = _pad_repeat ? n - 1 : (pos - n) % n;
            out.padded++;
        }
        const FileEntry& e = _all[_order[pos]];
        out.paths.push_back(e.path);
        out.names.push_back(e.name);
        out.labels.push_back(e.label);
        if (_with_boxes) {
            out.boxes.insert(out.boxes.end(), e.boxes.begin(), e.boxes.end());
            out.box_labels.insert(out.box_labels.end(), e.box_labels.begin(), e.box_labels.end());
            out.counts.push_back((int)e.box_labels.size());
        }
    }
    _cursor++;
    _last_padded = out.padded;
    return true;
}

void FileSource::reset() {
    _epoch++;
    begin_epoch();
}

}  // namespace rb200
