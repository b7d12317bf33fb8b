#include "coco_reader.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

namespace rb200 {

namespace {

// A small pull parser over a complete JSON text: just enough structure to walk objects and arrays, read numbers
// and strings, and skip whatever is not asked for.
class Json {
   public:
    explicit Json(const std::string& text) : _p(text.c_str()), _end(text.c_str() + text.size()) {}

    void ws() {
        while (_p < _end && (*_p == ' ' || *_p == '\n' || *_p == '\t' || *_p == '\r')) _p++;
    }
    char peek() {
        ws();
        if (_p >= _end) fail("unexpected end of file");
        return *_p;
    }
    void expect(char c) {
        if (peek() != c) fail(std::string("expected '") + c + "'");
        _p++;
    }
    bool accept(char c) {
        if (peek() == c) {
            _p++;
            return true;
        }
        return false;
    }
    std::string string() {
        expect('"');
        std::string out;
        while (_p < _end && *_p != '"') {
            if (*_p == '\\') {
                _p++;
                if (_p >= _end) fail("unterminated string");
                switch (*_p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        if (_end - _p < 5) fail("bad \\u escape");
                        unsigned cp = (unsigned)std::strtoul(std::string(_p + 1, _p + 5).c_str(), nullptr, 16);
                        _p += 4;
                        if (cp < 0x80) out += (char)cp;
                        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
                        else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
                        break;
                    }
                    default: out += *_p;   // \" \\ \/
                }
                _p++;
            } else {
                out += *_p++;
            }
        }
        if (_p >= _end) fail("unterminated string");
        _p++;
        return out;
    }
    double number() {
        ws();
        char* e = nullptr;
        double v = std::strtod(_p, &e);
        if (e == _p) fail("expected a number");
        _p = e;
        return v;
    }
    void skip() {
        char c = peek();
        if (c == '"') {
            string();
        } else if (c == '{') {
            _p++;
            if (accept('}')) return;
            do {
                string();
                expect(':');
                skip();
            } while (accept(','));
            expect('}');
        } else if (c == '[') {
            _p++;
            if (accept(']')) return;
            do skip();
            while (accept(','));
            expect(']');
        } else if (c == 't' || c == 'f' || c == 'n') {
            while (_p < _end && *_p >= 'a' && *_p <= 'z') _p++;
        } else {
            number();
        }
    }
    [[noreturn]] void fail(const std::string& what) { throw std::runtime_error("COCO annotations: " + what); }

   private:
    const char* _p;
    const char* _end;
};

}  // namespace

std::vector<CocoImage> read_coco_annotations(const std::string& json_path, bool avoid_class_remapping) {
    FILE* f = std::fopen(json_path.c_str(), "rb");
    if (!f) throw std::runtime_error("ERROR: Given annotations file not present " + json_path);
    std::fseek(f, 0, SEEK_END);
    long len = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    if (len <= 0) {
        std::fclose(f);
        throw std::runtime_error("ERROR: Given annotations file not valid " + json_path);
    }
    std::string text((size_t)len, '\0');
    size_t got = std::fread(&text[0], 1, (size_t)len, f);
    std::fclose(f);
    if (got != (size_t)len) throw std::runtime_error("short read on " + json_path);

    struct Ann {
        long image_id;
        int category;
        double bbox[4];
    };
    std::map<long, CocoImage> images;           // by image id
    std::map<int, int> class_index;             // category id -> 1-based index in order of appearance
    std::vector<Ann> anns;

    Json j(text);
    j.expect('{');
    if (!j.accept('}')) {
        do {
            const std::string key = j.string();
            j.expect(':');
            if (key == "images" || key == "categories" || key == "annotations") {
                j.expect('[');
                if (!j.accept(']')) {
                    do {
                        if (j.peek() != '{') {
                            j.skip();
                            continue;
                        }
                        j.expect('{');
                        long id = 1, image_id = 1;
                        int category = 0, width = 0, height = 0;
                        double bbox[4] = {0, 0, 0, 0};
                        std::string file_name;
                        if (!j.accept('}')) {
                            do {
                                const std::string k = j.string();
                                j.expect(':');
                                if (k == "id") id = (long)j.number();
                                else if (key == "images" && k == "file_name") file_name = j.string();
                                else if (key == "images" && k == "width") width = (int)j.number();
                                else if (key == "images" && k == "height") height = (int)j.number();
                                else if (key == "annotations" && k == "image_id") image_id = (long)j.number();
                                else if (key == "annotations" && k == "category_id") category = (int)j.number();
                                else if (key == "annotations" && k == "bbox") {
                                    j.expect('[');
                                    int n = 0;
                                    if (!j.accept(']')) {
                                        do {
                                            double v = j.number();
                                            if (n < 4) bbox[n] = v;
                                            n++;
                                        } while (j.accept(','));
                                        j.expect(']');
                                    }
                                } else {
                                    j.skip();
                                }
                            } while (j.accept(','));
                            j.expect('}');
                        }
                        if (key == "images") {
                            CocoImage im;
                            im.file_name = file_name;
                            im.id = id;
                            im.width = width;
                            im.height = height;
                            images[id] = im;
                        } else if (key == "categories") {
                            if (!class_index.count((int)id)) {
                                int next = (int)class_index.size() + 1;
                                class_index[(int)id] = next;
                            }
                        } else {
                            Ann a;
                            a.image_id = image_id;
                            a.category = category;
                            std::memcpy(a.bbox, bbox, sizeof(bbox));
                            anns.push_back(a);
                        }
                    } while (j.accept(','));
                    j.expect(']');
                }
            } else {
                j.skip();
            }
        } while (j.accept(','));
        j.expect('}');
    }

    // annotations may precede the images in the file: they are attached once everything is read
    for (const Ann& a : anns) {
        auto it = images.find(a.image_id);
        if (it == images.end()) continue;
        CocoImage& im = it->second;
        if (im.width <= 0 || im.height <= 0) continue;
        int label = a.category;
        if (!avoid_class_remapping) {
            auto c = class_index.find(a.category);
            if (c == class_index.end()) continue;   // category not declared
            label = c->second;
        }
        const float W = (float)im.width, H = (float)im.height;
        im.boxes.push_back((float)a.bbox[0] / W);
        im.boxes.push_back((float)a.bbox[1] / H);
        im.boxes.push_back((float)(a.bbox[0] + a.bbox[2]) / W);
        im.boxes.push_back((float)(a.bbox[1] + a.bbox[3]) / H);
        im.labels.push_back(label);
    }
    std::vector<CocoImage> out;
    for (auto& kv : images)
        if (!kv.second.file_name.empty()) out.push_back(std::move(kv.second));
    std::sort(out.begin(), out.end(), [](const CocoImage& a, const CocoImage& b) { return a.file_name < b.file_name; });
    if (out.empty()) throw std::runtime_error("COCO annotations: no images in " + json_path);
    return out;
}

}  // namespace rb200
