// Safetensors checkpoint reading for the host executor: what Weights::load does in the
// reference (src/models/qwen3_5/native/src/model.rs:239-315) - one file or the files named by
// model.safetensors.index.json, memory-mapped; the language model's tensors found under the
// first of the prefixes "model.language_model.", "model.", "" that has embed_tokens.weight;
// every one of them required to be bfloat16; uploaded into the model's arena by name.
// The file format: 8 bytes little-endian header length, a JSON object
// {name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}, then the data.
#include <fcntl.h>
#include <stdint.h>
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
    std::string str;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> fields;
    const Json* get(const char* key) const {
        for (const auto& f : fields)
            if (f.first == key) return &f.second;
        return nullptr;
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
                    case 'u': {  // keep the escape as text: tensor and file names are ASCII
                        out += "\\u";
                        break;
                    }
                    default: out += *p;
                }
                p++;
            } else {
                out += *p++;
            }
        }
        if (p >= end) ok = false;
        p++;
        return out;
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
        } else if (!strncmp(p, "true", std::min<size_t>(4, end - p))) {
            v.kind = Json::Bool, v.b = true, p += 4;
        } else if (!strncmp(p, "false", std::min<size_t>(5, end - p))) {
            v.kind = Json::Bool, p += 5;
        } else if (!strncmp(p, "null", std::min<size_t>(4, end - p))) {
            p += 4;
        } else {
            char* stop = nullptr;
            std::string text(p, std::min<size_t>(64, end - p));
            v.kind = Json::Number;
            v.num = strtod(text.c_str(), &stop);
            if (stop == text.c_str()) ok = false;
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
    for (const auto& field : root.fields) {
        if (field.first == "__metadata__") continue;
        const Json *dtype = field.second.get("dtype"), *shape = field.second.get("shape"),
                   *offs = field.second.get("data_offsets");
        if (!dtype || dtype->kind != Json::String || !shape || shape->kind != Json::Array || !offs ||
            offs->kind != Json::Array || offs->items.size() != 2)
            return S1_ERR_CHECKPOINT_FORMAT;
        View v;
        v.dtype = dtype->str;
        for (const Json& d : shape->items) v.shape.push_back((uint64_t)d.num);
        const uint64_t begin = (uint64_t)offs->items[0].num, stop = (uint64_t)offs->items[1].num;
        if (begin > stop || stop > data_bytes) return S1_ERR_CHECKPOINT_FORMAT;
        v.data = base + 8 + header + begin;
        v.bytes = stop - begin;
        f->tensors[field.first] = v;
    }
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
// tensor) and uploaded; tensors the decoder does not use (lm_head, vision tower, MTP) are
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
        size_t planned = 0;
        if (s1_model_tensor(model, t.first.c_str(), nullptr, &planned) != 0) continue;  // not part of the decoder
        if (t.second->dtype != "BF16") {
            copy_name(t.first, offender, offender_cap);
            return S1_ERR_CHECKPOINT_DTYPE;
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

}  // extern "C"
