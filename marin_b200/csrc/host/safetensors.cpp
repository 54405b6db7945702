// The safetensors container, host side, in C++: the header is read and checked here; the tensor bytes are mapped by
// the caller (marin_b200/weights/safetensors_io.py), which asks this file where each tensor lies.
//
// Layout (the same the reference parses, crates/loader/src/safetensors.rs:54-106): 8 bytes little-endian header
// length, a JSON header mapping tensor name to {"dtype", "shape", "data_offsets": [begin, end]} (offsets relative to the
// end of the header, "__metadata__" is skipped), then the raw little-endian tensor bytes.  A file that cannot be
// trusted is refused with one line that says why: too short, a header that does not fit the file ("partial
// download?", safetensors.rs:220-224), a header that is not JSON, an entry whose offsets do not match its shape and
// dtype or reach past the end of the file.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#define MBH_API extern "C" __attribute__((visibility("default")))

namespace {

// ---- a small JSON reader: enough for headers (objects, arrays, strings, numbers, true/false/null) ----------------------
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool boolean = false;
    double number = 0.0;
    bool integral = false;
    long long integer = 0;
    std::string text;
    std::vector<Json> items;                                  // array elements, or object values
    std::vector<std::string> keys;                            // object keys, in file order
};

class JsonReader {
  public:
    JsonReader(const char* p, size_t n) : p_(p), end_(p + n) {}
    bool parse(Json* out, std::string* err) {
        if (!value(out, 0)) { *err = err_; return false; }
        skip();
        if (p_ != end_) { *err = "trailing characters after the JSON value"; return false; }
        return true;
    }

  private:
    void skip() { while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_; }
    bool fail(const char* why) { err_ = why; return false; }
    bool literal(const char* word) {
        const size_t n = std::strlen(word);
        if ((size_t)(end_ - p_) < n || std::memcmp(p_, word, n) != 0) return fail("unknown literal");
        p_ += n;
        return true;
    }
    bool string(std::string* out) {
        ++p_;                                                  // the opening quote
        while (p_ < end_ && *p_ != '"') {
            unsigned char c = (unsigned char)*p_++;
            if (c < 0x20) return fail("control character in a string");
            if (c != '\\') { out->push_back((char)c); continue; }
            if (p_ >= end_) return fail("unfinished escape");
            const char e = *p_++;
            switch (e) {
                case '"': out->push_back('"'); break;
                case '\\': out->push_back('\\'); break;
                case '/': out->push_back('/'); break;
                case 'b': out->push_back('\b'); break;
                case 'f': out->push_back('\f'); break;
                case 'n': out->push_back('\n'); break;
                case 'r': out->push_back('\r'); break;
                case 't': out->push_back('\t'); break;
                case 'u': {
                    if (end_ - p_ < 4) return fail("unfinished \\u escape");
                    unsigned code = 0;
                    for (int i = 0; i < 4; ++i) {
                        const char h = *p_++;
                        code <<= 4;
                        if (h >= '0' && h <= '9') code |= (unsigned)(h - '0');
                        else if (h >= 'a' && h <= 'f') code |= (unsigned)(h - 'a' + 10);
                        else if (h >= 'A' && h <= 'F') code |= (unsigned)(h - 'A' + 10);
                        else return fail("bad \\u escape");
                    }
                    // UTF-8 of a code unit of the basic plane (surrogate pairs are kept as two units: names do not use them)
                    if (code < 0x80) out->push_back((char)code);
                    else if (code < 0x800) { out->push_back((char)(0xC0 | (code >> 6))); out->push_back((char)(0x80 | (code & 0x3F))); }
                    else { out->push_back((char)(0xE0 | (code >> 12))); out->push_back((char)(0x80 | ((code >> 6) & 0x3F))); out->push_back((char)(0x80 | (code & 0x3F))); }
                    break;
                }
                default: return fail("unknown escape");
            }
        }
        if (p_ >= end_) return fail("unfinished string");
        ++p_;                                                  // the closing quote
        return true;
    }
    bool number(Json* out) {
        const char* start = p_;
        if (p_ < end_ && *p_ == '-') ++p_;
        bool digits = false, integral = true;
        while (p_ < end_ && *p_ >= '0' && *p_ <= '9') { ++p_; digits = true; }
        if (p_ < end_ && *p_ == '.') { integral = false; ++p_; while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_; }
        if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false;
            ++p_;
            if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (!digits) return fail("a number was expected");
        const std::string text(start, p_);
        out->kind = Json::Number;
        out->number = std::strtod(text.c_str(), nullptr);
        out->integral = integral && text.size() <= 18;
        if (out->integral) out->integer = std::strtoll(text.c_str(), nullptr, 10);
        return true;
    }
    bool value(Json* out, int depth) {
        if (depth > 64) return fail("nested too deeply");
        skip();
        if (p_ >= end_) return fail("unexpected end");
        const char c = *p_;
        if (c == '{') {
            out->kind = Json::Object;
            ++p_;
            skip();
            if (p_ < end_ && *p_ == '}') { ++p_; return true; }
            for (;;) {
                skip();
                if (p_ >= end_ || *p_ != '"') return fail("an object key was expected");
                std::string key;
                if (!string(&key)) return false;
                skip();
                if (p_ >= end_ || *p_ != ':') return fail("`:` was expected");
                ++p_;
                Json item;
                if (!value(&item, depth + 1)) return false;
                out->keys.push_back(std::move(key));
                out->items.push_back(std::move(item));
                skip();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; return true; }
                return fail("`,` or `}` was expected");
            }
        }
        if (c == '[') {
            out->kind = Json::Array;
            ++p_;
            skip();
            if (p_ < end_ && *p_ == ']') { ++p_; return true; }
            for (;;) {
                Json item;
                if (!value(&item, depth + 1)) return false;
                out->items.push_back(std::move(item));
                skip();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; return true; }
                return fail("`,` or `]` was expected");
            }
        }
        if (c == '"') { out->kind = Json::String; return string(&out->text); }
        if (c == 't') { out->kind = Json::Bool; out->boolean = true; return literal("true"); }
        if (c == 'f') { out->kind = Json::Bool; out->boolean = false; return literal("false"); }
        if (c == 'n') { out->kind = Json::Null; return literal("null"); }
        return number(out);
    }
    const char* p_;
    const char* end_;
    std::string err_;
};

const Json* member(const Json& object, const char* key) {
    for (size_t i = 0; i < object.keys.size(); ++i)
        if (object.keys[i] == key) return &object.items[i];
    return nullptr;
}

// ---- the header ---------------------------------------------------------------------------------------------------------
struct Entry {
    std::string name, dtype;
    std::vector<long long> shape;
    long long begin = 0, end = 0;
};

struct Header {
    long long data_start = 0;
    std::vector<Entry> entries;
};

int dtype_bytes(const std::string& d) {
    if (d == "BF16" || d == "F16" || d == "I16") return 2;
    if (d == "F32" || d == "I32") return 4;
    if (d == "F64" || d == "I64") return 8;
    if (d == "I8" || d == "U8" || d == "BOOL") return 1;
    return 0;
}

const long long MAX_HEADER_BYTES = 100LL * 1024 * 1024;

bool read_header(const char* path, Header* out, std::string* err) {
    const std::string where(path);
    FILE* fh = std::fopen(path, "rb");
    if (fh == nullptr) { *err = where + ": cannot be opened"; return false; }
    std::fseek(fh, 0, SEEK_END);
    const long long size = std::ftell(fh);
    std::fseek(fh, 0, SEEK_SET);
    unsigned char len8[8];
    if (size < 8 || std::fread(len8, 1, 8, fh) != 8) {
        std::fclose(fh);
        *err = where + ": too short to hold a safetensors header (partial download?)";
        return false;
    }
    unsigned long long header_len = 0;
    for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | len8[i];
    if (header_len > (unsigned long long)MAX_HEADER_BYTES || 8 + (long long)header_len > size) {
        std::fclose(fh);
        *err = where + ": header of " + std::to_string(header_len) + " bytes does not fit the file (partial download?)";
        return false;
    }
    std::string text((size_t)header_len, '\0');
    if (header_len > 0 && std::fread(&text[0], 1, (size_t)header_len, fh) != (size_t)header_len) {
        std::fclose(fh);
        *err = where + ": the header could not be read (partial download?)";
        return false;
    }
    std::fclose(fh);
    Json root;
    std::string why;
    if (!JsonReader(text.data(), text.size()).parse(&root, &why)) { *err = where + ": header is not valid JSON: " + why; return false; }
    if (root.kind != Json::Object) { *err = where + ": header must be a JSON object"; return false; }
    out->data_start = 8 + (long long)header_len;
    const long long data_bytes = size - out->data_start;
    for (size_t i = 0; i < root.keys.size(); ++i) {
        const std::string& name = root.keys[i];
        if (name == "__metadata__") continue;
        const Json& e = root.items[i];
        const Json* dtype = e.kind == Json::Object ? member(e, "dtype") : nullptr;
        const Json* shape = e.kind == Json::Object ? member(e, "shape") : nullptr;
        const Json* offsets = e.kind == Json::Object ? member(e, "data_offsets") : nullptr;
        bool ok = dtype != nullptr && dtype->kind == Json::String && shape != nullptr && shape->kind == Json::Array &&
                  offsets != nullptr && offsets->kind == Json::Array && offsets->items.size() == 2;
        Entry entry;
        if (ok) {
            entry.name = name;
            entry.dtype = dtype->text;
            for (const Json& s : shape->items) {
                if (s.kind != Json::Number || !s.integral) { ok = false; break; }
                entry.shape.push_back(s.integer);
            }
            for (const Json& o : offsets->items)
                if (o.kind != Json::Number || !o.integral) ok = false;
        }
        if (!ok) { *err = where + ": malformed entry for tensor `" + name + "`"; return false; }
        entry.begin = offsets->items[0].integer;
        entry.end = offsets->items[1].integer;
        const int width = dtype_bytes(entry.dtype);
        if (width == 0) { *err = where + ": tensor `" + name + "` has unsupported dtype " + entry.dtype; return false; }
        // the number of elements, refusing a product that would not fit: no tensor holds more elements than the file
        // has bytes, so a size that pushes the product past that is a lie (and would overflow if multiplied on)
        long long count = 1;
        bool empty = false;
        for (long long s : entry.shape) {
            if (s < 0) { *err = where + ": tensor `" + name + "` has a negative size"; return false; }
            if (s == 0) empty = true;
        }
        if (empty) count = 0;
        else
            for (long long s : entry.shape) {
                if (count > (data_bytes > 0 ? data_bytes : 0) / s) {
                    *err = where + ": tensor `" + name + "`: its shape holds more elements than the file has bytes";
                    return false;
                }
                count *= s;
            }
        if (entry.begin < 0 || entry.end < entry.begin || entry.end - entry.begin != count * width) {
            *err = where + ": tensor `" + name + "`: offsets " + std::to_string(entry.begin) + ".." + std::to_string(entry.end) +
                   " do not match its shape and dtype " + entry.dtype;
            return false;
        }
        if (entry.end > data_bytes) {
            *err = where + ": tensor `" + name + "` ends at byte " + std::to_string(entry.end) + " but the file holds " +
                   std::to_string(data_bytes) + " (partial download?)";
            return false;
        }
        out->entries.push_back(std::move(entry));
    }
    return true;
}

void put(const std::string& s, char* out, int cap) {
    if (out != nullptr && cap > 0) std::snprintf(out, (size_t)cap, "%s", s.c_str());
}

}  // namespace

// Opens a file's header.  Returns a handle, or null with the reason in err.
MBH_API void* mbl_open(const char* path, char* err, int cap) {
    Header* h = new Header();
    std::string why;
    if (!read_header(path, h, &why)) {
        put(why, err, cap);
        delete h;
        return nullptr;
    }
    return h;
}
MBH_API void mbl_close(void* h) { delete static_cast<Header*>(h); }
MBH_API int mbl_count(void* h) { return (int)static_cast<Header*>(h)->entries.size(); }
MBH_API long long mbl_data_start(void* h) { return static_cast<Header*>(h)->data_start; }
// Entry i, in file order: name, dtype, shape (at most shape_cap sizes), byte range relative to the data start.
// Returns the number of dimensions, or -1 if i is out of range or a buffer is too small.
MBH_API int mbl_entry(void* h, int i, char* name, int name_cap, char* dtype, int dtype_cap, long long* shape, int shape_cap,
                      long long* begin, long long* end) {
    Header* header = static_cast<Header*>(h);
    if (i < 0 || i >= (int)header->entries.size()) return -1;
    const Entry& e = header->entries[i];
    if ((int)e.name.size() >= name_cap || (int)e.dtype.size() >= dtype_cap || (int)e.shape.size() > shape_cap) return -1;
    put(e.name, name, name_cap);
    put(e.dtype, dtype, dtype_cap);
    for (size_t k = 0; k < e.shape.size(); ++k) shape[k] = e.shape[k];
    *begin = e.begin;
    *end = e.end;
    return (int)e.shape.size();
}
