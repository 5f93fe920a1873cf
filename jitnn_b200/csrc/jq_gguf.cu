// GGUF file -> device weights: header, metadata and tensor table of a GGUF v2 / v3 file, read from a read-only memory
// mapping with every access bounds-checked, and the upload of a tensor's blocks straight from the mapping.
//
// What the reference's reader does (jitnn-gguf/.../GgufFile.java:100-175 open, :329-418 tensors, :420-573 value parsing;
// GgmlType.java:25-65 block geometry) and what its tests demand of hostile input (GgufFileTest.java:115-155): wrong magic,
// unsupported version, truncation, dimensions or offsets beyond 2^63, sizes that overflow, data outside the file or off
// the alignment grid, arrays nested deeper than a small limit - all are errors, never reads past the mapping.
// Host code only; compiled with the rest of the library.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "jq_common.cuh"

namespace {

constexpr uint32_t GGUF_MAGIC = 0x46554747u;  // "GGUF", little-endian
constexpr int MAX_ARRAY_DEPTH = 8;
constexpr int64_t DEFAULT_ALIGNMENT = 32;

// ggml type id -> values per block, bytes per block (0, 0: unknown id: the tensor is listed, its size is not known)
void geometry(int id, int* values, int* bytes) {
    static const int table[][3] = {{0, 1, 4},     {1, 1, 2},      {2, 32, 18},    {3, 32, 20},    {6, 32, 22},   {7, 32, 24},   {8, 32, 34},
                                   {9, 32, 36},   {10, 256, 84},  {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292},
                                   {24, 1, 1},    {25, 1, 2},     {26, 1, 4},     {27, 1, 8},     {28, 1, 8},    {30, 1, 2}};
    *values = *bytes = 0;
    for (const auto& row : table) {
        if (row[0] == id) {
            *values = row[1];
            *bytes = row[2];
        }
    }
}

struct MetaValue {
    int type;          // GGUF value type 0..12
    double number;     // numeric types and bool
    int64_t integer;   // integer types, exact
    int64_t pos, len;  // strings: position and length of the bytes in the file; arrays: element count in len
    int elem_type;     // arrays
};

struct TensorInfo {
    std::string name;
    int type, n_dims;
    int64_t dims[8];   // outermost first (GGUF stores the innermost first)
    int64_t offset;    // absolute, in the file
    int64_t nbytes;    // -1: unknown type
};

struct Truncated {};
struct Malformed {
    std::string what;
};

struct Reader {
    const uint8_t* p;
    int64_t size, pos;
    void need(int64_t n) const {
        if (n < 0 || n > size - pos) {
            throw Truncated{};
        }
    }
    template <typename T>
    T get() {
        need((int64_t)sizeof(T));
        T v;
        memcpy(&v, p + pos, sizeof(T));
        pos += (int64_t)sizeof(T);
        return v;
    }
    int64_t count(const char* what) {
        const uint64_t v = get<uint64_t>();
        if (v > (uint64_t)size) {  // every counted thing takes at least one byte of the file
            throw Malformed{std::string(what) + " " + std::to_string(v) + " exceeds the file"};
        }
        return (int64_t)v;
    }
    std::string str() {
        const int64_t n = count("string length");
        need(n);
        std::string s(reinterpret_cast<const char*>(p + pos), (size_t)n);
        pos += n;
        return s;
    }
    void skip_value(int type, int depth, MetaValue* out) {
        static const int width[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
        if (type < 0 || type > 12) {
            throw Malformed{"metadata value type " + std::to_string(type)};
        }
        if (type == 8) {
            const int64_t n = count("string length");
            need(n);
            if (out != nullptr) {
                out->pos = pos;
                out->len = n;
            }
            pos += n;
        } else if (type == 9) {
            if (depth >= MAX_ARRAY_DEPTH) {
                throw Malformed{"arrays nested deeper than " + std::to_string(MAX_ARRAY_DEPTH)};
            }
            const int et = (int)get<uint32_t>();
            const int64_t n = count("array length");
            if (out != nullptr) {
                out->elem_type = et;
                out->len = n;
            }
            if (et >= 0 && et <= 12 && width[et] > 0) {
                need(n * width[et]);  // n <= size, width <= 8: no overflow
                pos += n * width[et];
            } else {
                for (int64_t i = 0; i < n; i++) {
                    skip_value(et, depth + 1, nullptr);
                }
            }
        } else {
            need(width[type]);
            if (out != nullptr) {
                switch (type) {
                    case 0: out->integer = get<uint8_t>(); break;
                    case 1: out->integer = get<int8_t>(); break;
                    case 2: out->integer = get<uint16_t>(); break;
                    case 3: out->integer = get<int16_t>(); break;
                    case 4: out->integer = get<uint32_t>(); break;
                    case 5: out->integer = get<int32_t>(); break;
                    case 6: out->number = get<float>(); break;
                    case 7: out->integer = get<uint8_t>() != 0; break;
                    case 10: out->integer = (int64_t)get<uint64_t>(); break;
                    case 11: out->integer = get<int64_t>(); break;
                    default: out->number = get<double>(); break;
                }
                if (type != 6 && type != 12) {
                    out->number = (double)out->integer;
                }
            } else {
                pos += width[type];
            }
        }
    }
};

}  // namespace

struct jq_gguf {
    uint32_t magic;
    int fd;
    const uint8_t* map;
    int64_t size;
    int version;
    int64_t alignment, data_offset;
    std::vector<std::pair<std::string, MetaValue>> meta;
    std::vector<TensorInfo> tensors;
    std::map<std::string, int64_t> by_name;
};

#define JQ_GGUF_MAGIC 0x4a514746u

using namespace jq;

static int check_file(const jq_gguf* f, const char* who) {
    if (f == nullptr || f->magic != JQ_GGUF_MAGIC) {
        return fail(JQ_ERR_INVALID, "%s: not an open GGUF file handle", who);
    }
    return JQ_OK;
}

extern "C" {

JQ_API int jq_gguf_close(jq_gguf* f) {
    if (f == nullptr) {
        return JQ_OK;
    }
    int rc = check_file(f, "jq_gguf_close");
    if (rc != JQ_OK) {
        return rc;
    }
    if (f->map != nullptr && f->size > 0) {
        munmap(const_cast<uint8_t*>(f->map), (size_t)f->size);
    }
    if (f->fd >= 0) {
        close(f->fd);
    }
    f->magic = 0;
    delete f;
    return JQ_OK;
}

JQ_API int jq_gguf_open(const char* path, jq_gguf** out) {
    if (path == nullptr || out == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_gguf_open: null path or result pointer");
    }
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) {
        return fail(JQ_ERR_INVALID, "%s: cannot be opened (%s)", path, strerror(errno));
    }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) {
        close(fd);
        return fail(JQ_ERR_INVALID, "%s: not a GGUF file", path);
    }
    void* map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) {
        close(fd);
        return fail(JQ_ERR_INVALID, "%s: cannot be mapped (%s)", path, strerror(errno));
    }
    jq_gguf* f = new (std::nothrow) jq_gguf();
    if (f == nullptr) {
        munmap(map, (size_t)st.st_size);
        close(fd);
        return fail(JQ_ERR_OOM, "jq_gguf_open: out of host memory");
    }
    f->magic = JQ_GGUF_MAGIC;
    f->fd = fd;
    f->map = static_cast<const uint8_t*>(map);
    f->size = (int64_t)st.st_size;
    std::string problem;
    try {
        Reader r{f->map, f->size, 0};
        if (r.get<uint32_t>() != GGUF_MAGIC) {
            throw Malformed{"not a GGUF file"};
        }
        f->version = (int)r.get<uint32_t>();
        if (f->version != 2 && f->version != 3) {
            throw Malformed{"GGUF version " + std::to_string((uint32_t)f->version) + " is not supported (2 and 3 are; big-endian files are not)"};
        }
        const int64_t n_tensors = r.count("tensor count"), n_meta = r.count("metadata count");
        f->alignment = DEFAULT_ALIGNMENT;
        for (int64_t i = 0; i < n_meta; i++) {
            std::string key = r.str();
            MetaValue v{};
            v.type = (int)r.get<uint32_t>();
            r.skip_value(v.type, 0, &v);
            if (key == "general.alignment") {
                const bool integral = v.type <= 5 || v.type == 10 || v.type == 11;
                if (!integral || v.integer <= 0 || (v.integer & (v.integer - 1)) != 0) {
                    throw Malformed{"general.alignment is not a power of two"};
                }
                f->alignment = v.integer;
            }
            f->meta.emplace_back(std::move(key), v);
        }
        struct RawInfo {
            uint64_t dims[8];
            uint64_t offset;
        };
        std::vector<RawInfo> raw;
        for (int64_t i = 0; i < n_tensors; i++) {
            TensorInfo t{};
            t.name = r.str();
            const uint32_t nd = r.get<uint32_t>();
            if (nd > 8) {
                throw Malformed{"tensor " + t.name + " has " + std::to_string(nd) + " dimensions"};
            }
            t.n_dims = (int)nd;
            RawInfo ri{};
            for (uint32_t d = 0; d < nd; d++) {
                ri.dims[d] = r.get<uint64_t>();
            }
            t.type = (int)r.get<uint32_t>();
            ri.offset = r.get<uint64_t>();
            raw.push_back(ri);
            f->tensors.push_back(std::move(t));
        }
        f->data_offset = (r.pos + f->alignment - 1) / f->alignment * f->alignment;
        for (size_t i = 0; i < f->tensors.size(); i++) {
            TensorInfo& t = f->tensors[i];
            const RawInfo& ri = raw[i];
            if (ri.offset > (uint64_t)INT64_MAX - (uint64_t)f->data_offset) {
                throw Malformed{"tensor " + t.name + " has offset " + std::to_string(ri.offset)};
            }
            unsigned __int128 numel = 1;
            for (int d = 0; d < t.n_dims; d++) {
                const uint64_t dim = ri.dims[t.n_dims - 1 - d];  // GGUF lists the innermost axis first
                if (dim > (uint64_t)INT64_MAX) {
                    throw Malformed{"tensor " + t.name + " has dimension " + std::to_string(dim)};
                }
                t.dims[d] = (int64_t)dim;
                numel *= dim;
                if (numel > (unsigned __int128)INT64_MAX) {
                    throw Malformed{"the size of tensor " + t.name + " overflows"};
                }
            }
            int qk = 0, bb = 0;
            geometry(t.type, &qk, &bb);
            t.offset = f->data_offset + (int64_t)ri.offset;
            t.nbytes = -1;
            if (qk > 0) {
                const int64_t n = (int64_t)numel;
                const int64_t inner = t.n_dims > 0 ? t.dims[t.n_dims - 1] : 1;
                if (inner % qk != 0) {
                    throw Malformed{"tensor " + t.name + ": innermost dimension " + std::to_string(inner) + " is not a multiple of the block size " +
                                    std::to_string(qk)};
                }
                const unsigned __int128 bytes = (unsigned __int128)(n / qk) * (unsigned)bb;
                if (bytes > (unsigned __int128)INT64_MAX) {
                    throw Malformed{"the size of tensor " + t.name + " overflows"};
                }
                t.nbytes = (int64_t)bytes;
            }
            if (ri.offset % (uint64_t)f->alignment != 0 || t.offset > f->size || (t.nbytes >= 0 && t.nbytes > f->size - t.offset)) {
                throw Malformed{"tensor " + t.name + " lies outside the file or is not aligned"};
            }
            f->by_name[t.name] = (int64_t)i;
        }
    } catch (const Truncated&) {
        problem = "truncated GGUF file";
    } catch (const Malformed& m) {
        problem = m.what;
    } catch (const std::bad_alloc&) {
        problem = "out of host memory while reading the header";
    }
    if (!problem.empty()) {
        jq_gguf_close(f);
        return fail(JQ_ERR_INVALID, "%s: %s", path, problem.c_str());
    }
    *out = f;
    return JQ_OK;
}

JQ_API int jq_gguf_info(const jq_gguf* f, int* version, int64_t* alignment, int64_t* data_offset, int64_t* n_tensors, int64_t* n_meta) {
    int rc = check_file(f, "jq_gguf_info");
    if (rc != JQ_OK) {
        return rc;
    }
    if (version != nullptr) *version = f->version;
    if (alignment != nullptr) *alignment = f->alignment;
    if (data_offset != nullptr) *data_offset = f->data_offset;
    if (n_tensors != nullptr) *n_tensors = (int64_t)f->tensors.size();
    if (n_meta != nullptr) *n_meta = (int64_t)f->meta.size();
    return JQ_OK;
}

JQ_API int jq_gguf_tensor(const jq_gguf* f, int64_t index, const char** name, int* ggml_type, int* n_dims, int64_t* dims, int64_t* offset, int64_t* nbytes) {
    int rc = check_file(f, "jq_gguf_tensor");
    if (rc != JQ_OK) {
        return rc;
    }
    if (index < 0 || index >= (int64_t)f->tensors.size()) {
        return fail(JQ_ERR_INVALID, "jq_gguf_tensor: index %lld of %zu tensors", (long long)index, f->tensors.size());
    }
    const TensorInfo& t = f->tensors[(size_t)index];
    if (name != nullptr) *name = t.name.c_str();
    if (ggml_type != nullptr) *ggml_type = t.type;
    if (n_dims != nullptr) *n_dims = t.n_dims;
    if (dims != nullptr) {
        for (int d = 0; d < 8; d++) {
            dims[d] = d < t.n_dims ? t.dims[d] : 1;
        }
    }
    if (offset != nullptr) *offset = t.offset;
    if (nbytes != nullptr) *nbytes = t.nbytes;
    return JQ_OK;
}

JQ_API int jq_gguf_find_tensor(const jq_gguf* f, const char* name, int64_t* index) {
    int rc = check_file(f, "jq_gguf_find_tensor");
    if (rc != JQ_OK) {
        return rc;
    }
    if (name == nullptr || index == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_gguf_find_tensor: null name or result pointer");
    }
    auto it = f->by_name.find(name);
    if (it == f->by_name.end()) {
        return fail(JQ_ERR_INVALID, "no tensor %s", name);
    }
    *index = it->second;
    return JQ_OK;
}

JQ_API int jq_gguf_tensor_data(const jq_gguf* f, int64_t index, const void** data) {
    int rc = check_file(f, "jq_gguf_tensor_data");
    if (rc != JQ_OK) {
        return rc;
    }
    if (data == nullptr || index < 0 || index >= (int64_t)f->tensors.size()) {
        return fail(JQ_ERR_INVALID, "jq_gguf_tensor_data: index %lld of %zu tensors", (long long)index, f->tensors.size());
    }
    const TensorInfo& t = f->tensors[(size_t)index];
    if (t.nbytes < 0) {
        return fail(JQ_ERR_UNSUPPORTED, "%s: ggml type %d is unknown, so its size is too", t.name.c_str(), t.type);
    }
    *data = f->map + t.offset;
    return JQ_OK;
}

// Metadata: type of the value under `key` (GGUF value types 0..12; for arrays *array_len and *elem_type are set).
JQ_API int jq_gguf_meta_find(const jq_gguf* f, const char* key, int* value_type, int64_t* array_len, int* elem_type) {
    int rc = check_file(f, "jq_gguf_meta_find");
    if (rc != JQ_OK) {
        return rc;
    }
    for (const auto& kv : f->meta) {
        if (key != nullptr && kv.first == key) {
            if (value_type != nullptr) *value_type = kv.second.type;
            if (array_len != nullptr) *array_len = kv.second.type == 9 ? kv.second.len : 0;
            if (elem_type != nullptr) *elem_type = kv.second.type == 9 ? kv.second.elem_type : -1;
            return JQ_OK;
        }
    }
    return fail(JQ_ERR_INVALID, "no metadata key %s", key != nullptr ? key : "(null)");
}

JQ_API int jq_gguf_meta_number(const jq_gguf* f, const char* key, double* value, int64_t* integer) {
    int rc = check_file(f, "jq_gguf_meta_number");
    if (rc != JQ_OK) {
        return rc;
    }
    for (const auto& kv : f->meta) {
        if (key != nullptr && kv.first == key) {
            if (kv.second.type == 8 || kv.second.type == 9) {
                return fail(JQ_ERR_INVALID, "metadata key %s is not a number", key);
            }
            if (value != nullptr) *value = kv.second.number;
            if (integer != nullptr) *integer = (kv.second.type == 6 || kv.second.type == 12) ? (int64_t)kv.second.number : kv.second.integer;
            return JQ_OK;
        }
    }
    return fail(JQ_ERR_INVALID, "no metadata key %s", key != nullptr ? key : "(null)");
}

JQ_API int jq_gguf_meta_string(const jq_gguf* f, const char* key, const char** bytes, int64_t* length) {
    int rc = check_file(f, "jq_gguf_meta_string");
    if (rc != JQ_OK) {
        return rc;
    }
    for (const auto& kv : f->meta) {
        if (key != nullptr && kv.first == key) {
            if (kv.second.type != 8) {
                return fail(JQ_ERR_INVALID, "metadata key %s is not a string", key);
            }
            if (bytes != nullptr) *bytes = reinterpret_cast<const char*>(f->map + kv.second.pos);  // not NUL-terminated
            if (length != nullptr) *length = kv.second.len;
            return JQ_OK;
        }
    }
    return fail(JQ_ERR_INVALID, "no metadata key %s", key != nullptr ? key : "(null)");
}

// Rows [row_begin, row_end) of the 2-D quantised tensor `index` as a device weight, copied straight from the mapping
// (row_end = -1: all rows).
JQ_API int jq_gguf_upload(const jq_gguf* f, int64_t index, int device, int64_t row_begin, int64_t row_end, jq_weight** out) {
    int rc = check_file(f, "jq_gguf_upload");
    if (rc != JQ_OK) {
        return rc;
    }
    if (out == nullptr || index < 0 || index >= (int64_t)f->tensors.size()) {
        return fail(JQ_ERR_INVALID, "jq_gguf_upload: index %lld of %zu tensors", (long long)index, f->tensors.size());
    }
    const TensorInfo& t = f->tensors[(size_t)index];
    if (t.n_dims != 2 || t.nbytes < 0) {
        return fail(JQ_ERR_INVALID, "%s: a weight must be a 2-D tensor of a known type (it has %d dimensions, ggml type %d)", t.name.c_str(), t.n_dims, t.type);
    }
    const int64_t n = t.dims[0], k = t.dims[1];
    if (row_end < 0) {
        row_end = n;
    }
    return jq_weight_upload_rows(device, t.type, f->map + t.offset, t.nbytes, n, k, row_begin, row_end, JQ_LAYOUT_AUTO, out);
}

}  // extern "C"
