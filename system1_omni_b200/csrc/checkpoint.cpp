// Safetensors checkpoint reading for the host executor: what Weights::load does in the
// reference (src/models/qwen3_5/native/src/model.rs:239-315) - one file or the files named by
// model.safetensors.index.json, memory-mapped; the language model's tensors found under the
// first of the prefixes "model.language_model.", "model.", "" that has embed_tokens.weight;
// every one of them required to be bfloat16; uploaded into the model's arena by name.
// The file format: 8 bytes little-endian header length, a JSON object
// {name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}, then the data.
#include <errno.h>
#include <fcntl.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "s1_executor.h"

namespace {

// ---- a JSON reader sufficient for safetensors headers, their index and config files ----
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0;
    std::string str;  // a string's text, or a number's digits as written

    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> fields;
    const Json* get(const char* key) const {
        for (const auto& f : fields)
            if (f.first == key) return &f.second;
        return nullptr;
    }
    // A non-negative integer written without fraction or exponent (offsets and extents: exact
    // beyond 2^53, where a double is not).
    bool as_u64(uint64_t* out) const {
        if (kind != Number || str.empty()) return false;
        for (char ch : str)
            if (ch < '0' || ch > '9') return false;
        errno = 0;
        char* stop = nullptr;
        const unsigned long long v = strtoull(str.c_str(), &stop, 10);
        if (errno != 0 || *stop != 0) return false;
        *out = v;
        return true;
    }
};

struct Parser {
    const char* p;
    const char* end;
    bool ok = true;
    int depth = 0;
    void skip() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++;
    }
    bool eat(char c) {
        skip();
        if (p < end && *p == c) {
            p++;
            return true;
        }
        return false;
    }
    std::string string() {
        std::string out;
        if (!eat('"')) {
            ok = false;
            return out;
        }
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                p++;
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {  // four hex digits; code points up to 0x7ff become UTF-8, others stay escaped text
                        unsigned code = 0;
                        bool hex = end - p > 4;
                        for (int i = 1; hex && i <= 4; i++) {
                            const char ch = p[i];
                            const int d = ch >= '0' && ch <= '9' ? ch - '0' : ch >= 'a' && ch <= 'f' ? ch - 'a' + 10 : ch >= 'A' && ch <= 'F' ? ch - 'A' + 10 : -1;
                            if (d < 0) hex = false;
                            code = code * 16 + (unsigned)(d < 0 ? 0 : d);
                        }
                        if (!hex) {
                            ok = false;
                            return out;
                        }
                        if (code < 0x80) {
                            out += (char)code;
                        } else if (code < 0x800) {
                            out += (char)(0xc0 | (code >> 6));
                            out += (char)(0x80 | (code & 0x3f));
                        } else {
                            out.append(p - 1, 6);
                        }
                        p += 4;
                        break;
                    }
                    default: out += *p;
                }
                p++;
            } else {
                out += *p++;
            }
        }
        if (p >= end) {
            ok = false;
            return out;
        }
        p++;
        return out;
    }
    // A literal, whole: a header cut off inside one is malformed.
    bool literal(const char* word) {
        const size_t n = strlen(word);
        if ((size_t)(end - p) < n || strncmp(p, word, n) != 0) return false;
        p += n;
        return true;
    }
    Json value() {
        Json v;
        if (++depth > 64) {
            ok = false;
            return v;
        }
        skip();
        if (p >= end) {
            ok = false;
        } else if (*p == '{') {
            p++;
            v.kind = Json::Object;
            if (!eat('}')) {
                do {
                    std::string key = string();
                    if (!ok || !eat(':')) {
                        ok = false;
                        break;
                    }
                    v.fields.emplace_back(std::move(key), value());
                } while (ok && eat(','));
                if (ok && !eat('}')) ok = false;
            }
        } else if (*p == '[') {
            p++;
            v.kind = Json::Array;
            if (!eat(']')) {
                do v.items.push_back(value());
                while (ok && eat(','));
                if (ok && !eat(']')) ok = false;
            }
        } else if (*p == '"') {
            v.kind = Json::String;
            v.str = string();
        } else if (literal("true")) {
            v.kind = Json::Bool, v.b = true;
        } else if (literal("false")) {
            v.kind = Json::Bool;
        } else if (literal("null")) {
        } else {
            char* stop = nullptr;
            std::string text(p, std::min<size_t>(64, end - p));
            v.kind = Json::Number;
            v.num = strtod(text.c_str(), &stop);
            if (stop == text.c_str()) ok = false;
            v.str.assign(text.c_str(), stop - text.c_str());
            p += stop - text.c_str();
        }
        depth--;
        return v;
    }
};

bool parse_json(const char* text, size_t len, Json* out) {
    Parser ps{text, text + len};
    *out = ps.value();
    ps.skip();
    return ps.ok && ps.p == ps.end;
}

// ---- a memory-mapped safetensors file ----
struct View {
    std::string dtype;
    std::vector<uint64_t> shape;
    const unsigned char* data = nullptr;
    uint64_t bytes = 0;
};

struct File {
    void* map = MAP_FAILED;
    size_t size = 0;
    std::map<std::string, View> tensors;
    ~File() {
        if (map != MAP_FAILED) munmap(map, size);
    }
};

int open_file(const std::string& path, File* f) {
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) return S1_ERR_CHECKPOINT_IO;
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 8) {
        close(fd);
        return S1_ERR_CHECKPOINT_FORMAT;
    }
    f->size = (size_t)st.st_size;
    f->map = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (f->map == MAP_FAILED) return S1_ERR_CHECKPOINT_IO;
    const unsigned char* base = static_cast<const unsigned char*>(f->map);
    uint64_t header = 0;
    for (int i = 7; i >= 0; i--) header = header << 8 | base[i];
    if (header > f->size - 8) return S1_ERR_CHECKPOINT_FORMAT;
    Json root;
    if (!parse_json(reinterpret_cast<const char*>(base + 8), header, &root) || root.kind != Json::Object)
        return S1_ERR_CHECKPOINT_FORMAT;
    const uint64_t data_bytes = f->size - 8 - header;
    std::vector<std::pair<uint64_t, uint64_t>> spans;
    for (const auto& field : root.fields) {
        if (field.first == "__metadata__") continue;
        const Json *dtype = field.second.get("dtype"), *shape = field.second.get("shape"),
                   *offs = field.second.get("data_offsets");
        if (!dtype || dtype->kind != Json::String || !shape || shape->kind != Json::Array || !offs ||
            offs->kind != Json::Array || offs->items.size() != 2)
            return S1_ERR_CHECKPOINT_FORMAT;
        View v;
        v.dtype = dtype->str;
        for (const Json& d : shape->items) {
            uint64_t extent = 0;
            if (!d.as_u64(&extent)) return S1_ERR_CHECKPOINT_FORMAT;
            v.shape.push_back(extent);
        }
        uint64_t begin = 0, stop = 0;
        if (!offs->items[0].as_u64(&begin) || !offs->items[1].as_u64(&stop)) return S1_ERR_CHECKPOINT_FORMAT;
        if (begin > stop || stop > data_bytes) return S1_ERR_CHECKPOINT_FORMAT;
        v.data = base + 8 + header + begin;
        v.bytes = stop - begin;
        f->tensors[field.first] = v;
        if (stop > begin) spans.emplace_back(begin, stop);
    }
    // two tensors may not share bytes
    std::sort(spans.begin(), spans.end());
    for (size_t i = 1; i < spans.size(); i++)
        if (spans[i].first < spans[i - 1].second) return S1_ERR_CHECKPOINT_FORMAT;
    return 0;
}

bool read_text(const std::string& path, std::string* out) {
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) return false;
    char buf[65536];
    ssize_t n;
    while ((n = read(fd, buf, sizeof buf)) > 0) out->append(buf, (size_t)n);
    close(fd);
    return n == 0;
}

// The files of a checkpoint directory: those the index names (sorted, unique), else the single file.
int checkpoint_files(const std::string& dir, std::vector<std::string>* files) {
    std::string text;
    if (read_text(dir + "/model.safetensors.index.json", &text)) {
        Json root;
        if (!parse_json(text.data(), text.size(), &root)) return S1_ERR_CHECKPOINT_FORMAT;
        const Json* map = root.get("weight_map");
        if (!map || map->kind != Json::Object) return S1_ERR_CHECKPOINT_FORMAT;
        for (const auto& f : map->fields)
            if (f.second.kind == Json::String) files->push_back(f.second.str);
        std::sort(files->begin(), files->end());
        files->erase(std::unique(files->begin(), files->end()), files->end());
    } else {
        files->push_back("model.safetensors");
    }
    return files->empty() ? S1_ERR_CHECKPOINT_FORMAT : 0;
}

struct Checkpoint {
    std::vector<std::unique_ptr<File>> files;
    std::string prefix;
    std::vector<std::pair<std::string, const View*>> ours;  // names without the prefix
};

int open_checkpoint(const char* dir, Checkpoint* ck) {
    std::vector<std::string> names;
    int rc = checkpoint_files(dir, &names);
    if (rc != 0) return rc;
    for (const std::string& n : names) {
        ck->files.emplace_back(new File());
        rc = open_file(std::string(dir) + "/" + n, ck->files.back().get());
        if (rc != 0) return rc;
    }
    bool found = false;
    for (const char* p : {"model.language_model.", "model.", ""}) {
        for (const auto& f : ck->files)
            if (f->tensors.count(std::string(p) + "embed_tokens.weight")) found = true;
        if (found) {
            ck->prefix = p;
            break;
        }
    }
    if (!found) return S1_ERR_CHECKPOINT_MISSING;
    for (const auto& f : ck->files)
        for (const auto& t : f->tensors)
            if (t.first.compare(0, ck->prefix.size(), ck->prefix) == 0)
                ck->ours.emplace_back(t.first.substr(ck->prefix.size()), &t.second);
    return 0;
}

void copy_name(const std::string& name, char* out, size_t cap) {
    if (!out || cap == 0) return;
    const size_t n = std::min(cap - 1, name.size());
    memcpy(out, name.data(), n);
    out[n] = 0;
}

}  // namespace

extern "C" {

// Lists a checkpoint without touching a GPU: the prefix found and the number of language-model
// tensors; with index >= 0 also that tensor's name (without the prefix), dtype, rank, shape and bytes.
int s1_checkpoint_inspect(const char* dir, char* prefix_out, size_t prefix_cap, int* n_tensors, int index,
                          char* name_out, size_t name_cap, char* dtype_out, size_t dtype_cap, int* rank,
                          uint64_t* shape8, uint64_t* bytes) {
    if (!dir) return S1_ERR_ARGUMENT;
    Checkpoint ck;
    const int rc = open_checkpoint(dir, &ck);
    if (rc != 0) return rc;
    copy_name(ck.prefix, prefix_out, prefix_cap);
    if (n_tensors) *n_tensors = (int)ck.ours.size();
    if (index >= 0) {
        if (index >= (int)ck.ours.size()) return S1_ERR_ARGUMENT;
        const View& v = *ck.ours[index].second;
        copy_name(ck.ours[index].first, name_out, name_cap);
        copy_name(v.dtype, dtype_out, dtype_cap);
        if (rank) *rank = (int)v.shape.size();
        for (size_t i = 0; shape8 && i < v.shape.size() && i < 8; i++) shape8[i] = v.shape[i];
        if (bytes) *bytes = v.bytes;
    }
    return 0;
}

// Model::load's weight half (model.rs:239-315, 622-705): every language-model tensor of the
// checkpoint that the model has a place for is checked (bfloat16, byte size of the planned
// tensor's shape) and uploaded; tensors the decoder does not use (lm_head, MTP) are
// skipped. Fails with S1_ERR_CHECKPOINT_DTYPE / S1_ERR_TENSOR_SIZE at the first offender
// and S1_ERR_CHECKPOINT_MISSING when a planned tensor is absent; `offender` (nullable) receives
// the tensor's name.
int s1_model_load_checkpoint(void* model, const char* dir, char* offender, size_t offender_cap) {
    if (!model || !dir) return S1_ERR_ARGUMENT;
    if (offender && offender_cap) offender[0] = 0;
    Checkpoint ck;
    int rc = open_checkpoint(dir, &ck);
    if (rc != 0) return rc;
    for (const auto& t : ck.ours) {
        // every tensor under the prefix must be bfloat16, used or not (model.rs:291-295)
        if (t.second->dtype != "BF16") {
            copy_name(t.first, offender, offender_cap);
            return S1_ERR_CHECKPOINT_DTYPE;
        }
        int rank = 0;
        uint64_t want[8] = {};
        if (s1_model_tensor_shape(model, t.first.c_str(), &rank, want) != 0) continue;  // not part of the decoder
        // the shape the decoder expects, not merely its byte count (model.rs:306-320): a transposed
        // matrix has the same bytes
        uint64_t elems = 1;
        bool same = (size_t)rank == t.second->shape.size();
        for (int i = 0; same && i < rank; i++) {
            same = want[i] == t.second->shape[i];
            elems *= want[i];
        }
        if (!same || elems * 2 != t.second->bytes) {
            copy_name(t.first, offender, offender_cap);
            return S1_ERR_TENSOR_SIZE;
        }
        rc = s1_model_set_tensor(model, t.first.c_str(), t.second->data, (size_t)t.second->bytes);
        if (rc != 0) {
            copy_name(t.first, offender, offender_cap);
            return rc;
        }
    }
    char missing[256];
    if (s1_model_unfilled(model, missing, sizeof missing) > 0) {
        copy_name(missing, offender, offender_cap);
        return S1_ERR_CHECKPOINT_MISSING;
    }
    return 0;
}

// The export manifest of a merged Open-Jev checkpoint, open_jev_export.json (written last by
// recipe/open_jev/export_merged.py:82-90; read by Engine::load, engine.rs:21-46, and
// DecisionHead::load, executor.rs:21-54): format tag, calibration temperature (finite, > 0),
// max_length (1..=16384), chat prefix and suffix (strings; the processor's business), and the
// trained scalar head - `hidden` finite weights and a finite bias, float64 in the file, rounded
// to float32 as the reference does. Host only. Every out pointer but head_weight is nullable.
int s1_export_read(const char* dir, int hidden, float* head_weight, float* head_bias, double* temperature,
                   int* max_length, char* model_id, size_t model_id_cap) {
    if (!dir || hidden <= 0 || !head_weight) return S1_ERR_ARGUMENT;
    std::string text;
    if (!read_text(std::string(dir) + "/open_jev_export.json", &text)) return S1_ERR_CHECKPOINT_IO;
    Json root;
    if (!parse_json(text.data(), text.size(), &root) || root.kind != Json::Object) return S1_ERR_CHECKPOINT_FORMAT;
    const Json* format = root.get("format");
    if (!format || format->kind != Json::String || format->str != "open-jev-text-merged/1") return S1_ERR_CHECKPOINT_FORMAT;
    const Json *temp = root.get("temperature"), *len = root.get("max_length"), *w = root.get("head_weight"),
               *b = root.get("head_bias"), *pre = root.get("chat_prefix"), *suf = root.get("chat_suffix"),
               *id = root.get("model_id");
    if (!temp || temp->kind != Json::Number || !isfinite(temp->num) || !(temp->num > 0.0)) return S1_ERR_EXPORT_FIELD;
    uint64_t max_len = 0;
    if (!len || !len->as_u64(&max_len) || max_len < 1 || max_len > 16384) return S1_ERR_EXPORT_FIELD;
    if (!pre || pre->kind != Json::String || !suf || suf->kind != Json::String) return S1_ERR_EXPORT_FIELD;
    if (!w || w->kind != Json::Array || (int)w->items.size() != hidden || !b || b->kind != Json::Number)
        return S1_ERR_EXPORT_FIELD;
    const float bias = (float)b->num;
    if (!isfinite(bias)) return S1_ERR_EXPORT_FIELD;
    for (int i = 0; i < hidden; i++) {
        const Json& x = w->items[i];
        if (x.kind != Json::Number) return S1_ERR_EXPORT_FIELD;
        const float v = (float)x.num;
        if (!isfinite(v)) return S1_ERR_EXPORT_FIELD;
        head_weight[i] = v;
    }
    if (head_bias) *head_bias = bias;
    if (temperature) *temperature = temp->num;
    if (max_length) *max_length = (int)max_len;
    if (model_id && model_id_cap) copy_name(id && id->kind == Json::String ? id->str : std::string(), model_id, model_id_cap);
    return 0;
}

}  // extern "C"
