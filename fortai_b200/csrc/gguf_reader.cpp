// GGUF v3 reader over a read-only memory mapping; see include/fortai_gguf_b200.h for the
// reference code each entry point stands for (src/fortai_gguf_runtime.f90).
#include "../../include/fortai_gguf_b200.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "../../include/fortai_cuda_backend_b200.h"

namespace {

enum GgufType : int32_t {
    kU8 = 0, kI8 = 1, kU16 = 2, kI16 = 3, kU32 = 4, kI32 = 5, kF32 = 6, kBool = 7, kString = 8,
    kArray = 9, kU64 = 10, kI64 = 11, kF64 = 12
};

struct Meta {
    std::string key;
    int32_t type = -1;
    int64_t integer = 0;
    float real = 0.0f;
    bool logical = false;
    const char *text = nullptr;     // inside the mapping
    int64_t text_bytes = 0;
    int32_t element_type = -1;
    std::vector<int64_t> integers;
    bool has_integers = false;
};

struct Tensor {
    std::string name;
    int32_t rank = 0;
    int64_t shape[4] = {1, 1, 1, 1};
    int32_t type = -1;
    int64_t file_offset = 0;
    int64_t byte_count = 0;
};

}  // namespace

struct fortai_gguf_file {
    int fd = -1;
    const uint8_t *base = nullptr;
    size_t size = 0;
    int32_t version = 0;
    int64_t tensor_count = 0;
    int64_t metadata_count = 0;
    int64_t alignment = 32;
    int64_t data_start = 0;
    std::vector<Meta> metadata;
    std::vector<Tensor> tensors;
};

namespace {

// Sequential reader over the mapping; `ok` turns false at the first short read, as the
// reference's iostat does.
struct Cursor {
    const uint8_t *base;
    size_t size;
    size_t at = 0;
    bool ok = true;

    template <typename T>
    T get() {
        T value{};
        if (!ok || size - at < sizeof(T) || at > size) {
            ok = false;
            return value;
        }
        std::memcpy(&value, base + at, sizeof(T));
        at += sizeof(T);
        return value;
    }

    // length-prefixed string: pointer into the mapping
    bool string(const char **text, int64_t *bytes) {
        const int64_t length = get<int64_t>();
        if (!ok || length < 0 || static_cast<uint64_t>(length) > size - at) {
            ok = false;
            return false;
        }
        *text = reinterpret_cast<const char *>(base + at);
        *bytes = length;
        at += static_cast<size_t>(length);
        return true;
    }
};

bool skip_value(Cursor &in, int32_t type) {
    switch (type) {
    case kU8: case kI8: case kBool: in.get<uint8_t>(); break;
    case kU16: case kI16: in.get<uint16_t>(); break;
    case kU32: case kI32: case kF32: in.get<uint32_t>(); break;
    case kU64: case kI64: case kF64: in.get<uint64_t>(); break;
    case kString: {
        const char *text;
        int64_t bytes;
        in.string(&text, &bytes);
        break;
    }
    default: in.ok = false;
    }
    return in.ok;
}

bool read_value(Cursor &in, int32_t type, Meta &m) {
    switch (type) {
    case kU8: m.integer = in.get<uint8_t>(); break;
    case kI8: m.integer = in.get<int8_t>(); break;
    case kU16: m.integer = in.get<uint16_t>(); break;
    case kI16: m.integer = in.get<int16_t>(); break;
    case kU32: m.integer = in.get<uint32_t>(); break;
    case kI32: m.integer = in.get<int32_t>(); break;
    case kU64: case kI64: m.integer = in.get<int64_t>(); break;
    case kF32: m.real = in.get<float>(); break;
    case kF64: m.real = static_cast<float>(in.get<double>()); break;
    case kBool: m.logical = in.get<uint8_t>() != 0; break;
    case kString: in.string(&m.text, &m.text_bytes); break;
    case kArray: {
        m.element_type = in.get<int32_t>();
        const int64_t count = in.get<int64_t>();
        if (!in.ok || count < 0) {
            in.ok = false;
            break;
        }
        const bool keep = m.element_type == kI32 || m.element_type == kU32 ||
            m.element_type == kI64 || m.element_type == kU64;
        if (keep) {
            // every element needs at least four bytes: refuse counts the file cannot hold
            if (static_cast<uint64_t>(count) > (in.size - in.at) / 4) {
                in.ok = false;
                break;
            }
            m.has_integers = true;
            m.integers.reserve(static_cast<size_t>(count));
            for (int64_t i = 0; i < count && in.ok; ++i) {
                // 32-bit elements are read as signed, as the reference does for both kinds
                if (m.element_type == kI32 || m.element_type == kU32)
                    m.integers.push_back(in.get<int32_t>());
                else
                    m.integers.push_back(in.get<int64_t>());
            }
        } else {
            for (int64_t i = 0; i < count && in.ok; ++i) skip_value(in, m.element_type);
        }
        break;
    }
    default: in.ok = false;
    }
    return in.ok;
}

// Product of the shape; false when it does not fit 63 bits (a file cannot hold such a tensor,
// and a wrapped product would pass the range check against the file size).
bool element_count(const Tensor &t, int64_t *count) {
    int64_t n = 1;
    for (int i = 0; i < t.rank; ++i)
        if (t.shape[i] < 0 || __builtin_mul_overflow(n, t.shape[i], &n)) return false;
    *count = n;
    return true;
}

int64_t element_count(const Tensor &t) {
    int64_t n = 0;
    return element_count(t, &n) ? n : 0;
}

// Size of a tensor's data; the reference's rules and messages.
int tensor_bytes(const Tensor &t, int64_t *bytes, const char **why) {
    int64_t elements = 0;
    if (!element_count(t, &elements)) {
        *why = "GGUF tensor shape overflows";
        return FORTAI_GGUF_INVALID;
    }
    switch (t.type) {
    case FORTAI_GGML_TYPE_F32:
        if (__builtin_mul_overflow(elements, static_cast<int64_t>(4), bytes)) break;
        return FORTAI_GGUF_OK;
    case FORTAI_GGML_TYPE_F16:
        if (__builtin_mul_overflow(elements, static_cast<int64_t>(2), bytes)) break;
        return FORTAI_GGUF_OK;
    case FORTAI_GGML_TYPE_Q8_0:
        if (t.shape[0] <= 0 || t.shape[0] % 32 != 0) {
            *why = "Q8_0 tensor width is not a multiple of 32";
            return FORTAI_GGUF_INVALID;
        }
        // blocks * 34 <= elements * 34 / 32: check the larger product
        if (__builtin_mul_overflow(elements / 32, static_cast<int64_t>(34), bytes)) break;
        return FORTAI_GGUF_OK;
    default:
        *why = "GGUF tensor quantization is not supported";
        return FORTAI_GGUF_UNSUPPORTED;
    }
    *why = "GGUF tensor shape overflows";
    return FORTAI_GGUF_INVALID;
}

float half_to_float(uint16_t raw) {
    const int exponent = (raw >> 10) & 31, fraction = raw & 1023;
    float value;
    if (exponent == 0) value = std::ldexp(static_cast<float>(fraction) / 1024.0f, -14);
    else if (exponent == 31) value = 3.402823466e+38f;        // huge(1.0), not inf / nan
    else value = std::ldexp(1.0f + static_cast<float>(fraction) / 1024.0f, exponent - 15);
    return (raw & 0x8000) ? -value : value;
}

int fail(char *message, size_t message_bytes, int code, const char *text) {
    if (message && message_bytes) std::snprintf(message, message_bytes, "%s", text);
    return code;
}

const Meta *find_meta(const fortai_gguf_file *file, const char *key) {
    if (!file || !key) return nullptr;
    for (const Meta &m : file->metadata)
        if (m.key == key) return &m;
    return nullptr;
}

bool is_integer_kind(int32_t type) {
    return type == kU8 || type == kI8 || type == kU16 || type == kI16 || type == kU32 ||
        type == kI32 || type == kU64 || type == kI64;
}

}  // namespace

extern "C" int fortai_gguf_open(const char *path, fortai_gguf_file **file, char *message,
    size_t message_bytes) {
    if (!file) return FORTAI_GGUF_INVALID;
    *file = nullptr;
    if (message && message_bytes) message[0] = '\0';
    if (!path) return fail(message, message_bytes, FORTAI_GGUF_INVALID, "no GGUF path");
    const int fd = ::open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return fail(message, message_bytes, FORTAI_GGUF_IO_ERROR, "could not open GGUF model");
    struct stat info;
    if (::fstat(fd, &info) != 0 || info.st_size <= 0) {
        ::close(fd);
        return fail(message, message_bytes, FORTAI_GGUF_INVALID, "unsupported or malformed GGUF header");
    }
    void *mapping = ::mmap(nullptr, static_cast<size_t>(info.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    if (mapping == MAP_FAILED) {
        ::close(fd);
        return fail(message, message_bytes, FORTAI_GGUF_IO_ERROR, "could not open GGUF model");
    }
    fortai_gguf_file *created = new (std::nothrow) fortai_gguf_file;
    if (!created) {
        ::munmap(mapping, static_cast<size_t>(info.st_size));
        ::close(fd);
        return fail(message, message_bytes, FORTAI_GGUF_OUT_OF_MEMORY, "out of memory");
    }
    created->fd = fd;
    created->base = static_cast<const uint8_t *>(mapping);
    created->size = static_cast<size_t>(info.st_size);
    auto give_up = [&](int code, const char *text) {
        fortai_gguf_close(created);
        return fail(message, message_bytes, code, text);
    };

    Cursor in{created->base, created->size};
    char magic[4] = {};
    for (char &c : magic) c = static_cast<char>(in.get<uint8_t>());
    created->version = in.get<int32_t>();
    created->tensor_count = in.get<int64_t>();
    created->metadata_count = in.get<int64_t>();
    if (!in.ok || std::memcmp(magic, "GGUF", 4) != 0 || created->version != 3)
        return give_up(FORTAI_GGUF_INVALID, "unsupported or malformed GGUF header");
    if (created->tensor_count < 0 || created->metadata_count < 0)
        return give_up(FORTAI_GGUF_INVALID, "GGUF counts cannot be negative");
    // an entry is at least twelve bytes: counts the file cannot hold are malformed, not a
    // reason to allocate
    if (static_cast<uint64_t>(created->metadata_count) > created->size / 12 ||
        static_cast<uint64_t>(created->tensor_count) > created->size / 12)
        return give_up(FORTAI_GGUF_IO_ERROR, "could not read GGUF metadata");
    try {
        created->metadata.resize(static_cast<size_t>(created->metadata_count));
        for (Meta &m : created->metadata) {
            const char *text = nullptr;
            int64_t bytes = 0;
            if (in.string(&text, &bytes)) m.key.assign(text, static_cast<size_t>(bytes));
            m.type = in.get<int32_t>();
            if (!in.ok || !read_value(in, m.type, m))
                return give_up(FORTAI_GGUF_IO_ERROR, "could not read GGUF metadata");
        }
        created->alignment = fortai_gguf_meta_int(created, "general.alignment", 32);
        if (created->alignment <= 0) created->alignment = 32;
        // a power of two of at most 1 MiB: anything else cannot be a GGUF alignment, and a huge
        // value would overflow the rounding of the data offset below
        if ((created->alignment & (created->alignment - 1)) != 0 || created->alignment > (1 << 20))
            return give_up(FORTAI_GGUF_INVALID, "invalid GGUF alignment");
        created->tensors.resize(static_cast<size_t>(created->tensor_count));
        for (Tensor &t : created->tensors) {
            const char *text = nullptr;
            int64_t bytes = 0;
            if (in.string(&text, &bytes)) t.name.assign(text, static_cast<size_t>(bytes));
            const int32_t rank = in.get<int32_t>();
            if (!in.ok || rank <= 0 || rank > 4)
                return give_up(FORTAI_GGUF_INVALID, "invalid GGUF tensor rank");
            t.rank = rank;
            for (int j = 0; j < rank; ++j) t.shape[j] = in.get<int64_t>();
            t.type = in.get<int32_t>();
            t.file_offset = in.get<int64_t>();
            if (!in.ok) return give_up(FORTAI_GGUF_IO_ERROR, "could not read GGUF tensor index");
            for (int j = 0; j < rank; ++j)
                if (t.shape[j] < 0) return give_up(FORTAI_GGUF_INVALID, "invalid GGUF tensor rank");
            const char *why = "";
            const int code = tensor_bytes(t, &t.byte_count, &why);
            if (code != FORTAI_GGUF_OK) return give_up(code, why);
        }
    } catch (const std::bad_alloc &) {
        return give_up(FORTAI_GGUF_OUT_OF_MEMORY, "out of memory");
    }
    const int64_t position = static_cast<int64_t>(in.at);
    created->data_start = (position + created->alignment - 1) / created->alignment *
        created->alignment;
    for (const Tensor &t : created->tensors) {
        const int64_t begin = created->data_start + t.file_offset;
        if (t.file_offset < 0 || begin < 0 || t.byte_count < 0 ||
            static_cast<uint64_t>(begin) > created->size ||
            static_cast<uint64_t>(t.byte_count) > created->size - static_cast<uint64_t>(begin))
            return give_up(FORTAI_GGUF_IO_ERROR, "could not read GGUF tensor data");
    }
    *file = created;
    return FORTAI_GGUF_OK;
}

extern "C" void fortai_gguf_close(fortai_gguf_file *file) {
    if (!file) return;
    if (file->base) ::munmap(const_cast<uint8_t *>(file->base), file->size);
    if (file->fd >= 0) ::close(file->fd);
    delete file;
}

extern "C" int32_t fortai_gguf_version(const fortai_gguf_file *file) {
    return file ? file->version : 0;
}
extern "C" int64_t fortai_gguf_tensor_count(const fortai_gguf_file *file) {
    return file ? file->tensor_count : 0;
}
extern "C" int64_t fortai_gguf_metadata_count(const fortai_gguf_file *file) {
    return file ? file->metadata_count : 0;
}
extern "C" int64_t fortai_gguf_alignment(const fortai_gguf_file *file) {
    return file ? file->alignment : 32;
}
extern "C" int64_t fortai_gguf_data_start(const fortai_gguf_file *file) {
    return file ? file->data_start : 0;
}

extern "C" int64_t fortai_gguf_find_meta(const fortai_gguf_file *file, const char *key) {
    if (!file || !key) return -1;
    for (size_t i = 0; i < file->metadata.size(); ++i)
        if (file->metadata[i].key == key) return static_cast<int64_t>(i);
    return -1;
}

extern "C" int64_t fortai_gguf_find_tensor(const fortai_gguf_file *file, const char *name) {
    if (!file || !name) return -1;
    for (size_t i = 0; i < file->tensors.size(); ++i)
        if (file->tensors[i].name == name) return static_cast<int64_t>(i);
    return -1;
}

extern "C" const char *fortai_gguf_meta_key(const fortai_gguf_file *file, int64_t index) {
    if (!file || index < 0 || index >= static_cast<int64_t>(file->metadata.size())) return nullptr;
    return file->metadata[static_cast<size_t>(index)].key.c_str();
}

extern "C" int32_t fortai_gguf_meta_type(const fortai_gguf_file *file, int64_t index) {
    if (!file || index < 0 || index >= static_cast<int64_t>(file->metadata.size())) return -1;
    return file->metadata[static_cast<size_t>(index)].type;
}

extern "C" int64_t fortai_gguf_meta_int(const fortai_gguf_file *file, const char *key,
    int64_t fallback) {
    const Meta *m = find_meta(file, key);
    return m && is_integer_kind(m->type) ? m->integer : fallback;
}

extern "C" float fortai_gguf_meta_real(const fortai_gguf_file *file, const char *key,
    float fallback) {
    const Meta *m = find_meta(file, key);
    return m && (m->type == kF32 || m->type == kF64) ? m->real : fallback;
}

extern "C" const char *fortai_gguf_meta_string(const fortai_gguf_file *file, const char *key,
    int64_t *length) {
    const Meta *m = find_meta(file, key);
    if (!m || m->type != kString) return nullptr;
    if (length) *length = m->text_bytes;
    return m->text;
}

extern "C" int fortai_gguf_meta_bool(const fortai_gguf_file *file, const char *key, int fallback) {
    const Meta *m = find_meta(file, key);
    return m && m->type == kBool ? (m->logical ? 1 : 0) : fallback;
}

extern "C" int64_t fortai_gguf_meta_int_array(const fortai_gguf_file *file, const char *key,
    int64_t *values, int64_t capacity) {
    const Meta *m = find_meta(file, key);
    if (!m || m->type != kArray || !m->has_integers) return -1;
    const int64_t count = static_cast<int64_t>(m->integers.size());
    if (values)
        for (int64_t i = 0; i < count && i < capacity; ++i) values[i] = m->integers[static_cast<size_t>(i)];
    return count;
}

extern "C" int fortai_gguf_tensor_info(const fortai_gguf_file *file, int64_t index,
    const char **name, int32_t *type, int32_t *rank, int64_t shape[4], int64_t *file_offset,
    int64_t *byte_count) {
    if (!file || index < 0 || index >= static_cast<int64_t>(file->tensors.size()))
        return FORTAI_GGUF_INVALID;
    const Tensor &t = file->tensors[static_cast<size_t>(index)];
    if (name) *name = t.name.c_str();
    if (type) *type = t.type;
    if (rank) *rank = t.rank;
    if (shape)
        for (int j = 0; j < 4; ++j) shape[j] = t.shape[j];
    if (file_offset) *file_offset = t.file_offset;
    if (byte_count) *byte_count = t.byte_count;
    return FORTAI_GGUF_OK;
}

extern "C" const void *fortai_gguf_tensor_data(const fortai_gguf_file *file, int64_t index) {
    if (!file || index < 0 || index >= static_cast<int64_t>(file->tensors.size())) return nullptr;
    return file->base + file->data_start + file->tensors[static_cast<size_t>(index)].file_offset;
}

extern "C" float fortai_gguf_tensor_value(const fortai_gguf_file *file, int64_t index,
    int64_t element) {
    if (!file || index < 0 || index >= static_cast<int64_t>(file->tensors.size())) return 0.0f;
    const Tensor &t = file->tensors[static_cast<size_t>(index)];
    if (element < 0 || element >= element_count(t)) return 0.0f;
    const uint8_t *bytes = file->base + file->data_start + t.file_offset;
    switch (t.type) {
    case FORTAI_GGML_TYPE_F32: {
        float v;
        std::memcpy(&v, bytes + 4 * element, 4);
        return v;
    }
    case FORTAI_GGML_TYPE_F16: {
        uint16_t raw;
        std::memcpy(&raw, bytes + 2 * element, 2);
        return half_to_float(raw);
    }
    case FORTAI_GGML_TYPE_Q8_0: {
        const uint8_t *block = bytes + (element / 32) * 34;
        uint16_t raw;
        std::memcpy(&raw, block, 2);
        return half_to_float(raw) * static_cast<float>(static_cast<int8_t>(block[2 + element % 32]));
    }
    default: return 0.0f;
    }
}

extern "C" int fortai_gguf_tensor_get_row(const fortai_gguf_file *file, int64_t index, int64_t row,
    float *values, int64_t count) {
    if (!file || !values || index < 0 || index >= static_cast<int64_t>(file->tensors.size()))
        return FORTAI_GGUF_INVALID;
    const Tensor &t = file->tensors[static_cast<size_t>(index)];
    if (t.rank != 2) return FORTAI_GGUF_INVALID;             // "GGUF tensor is not a matrix"
    const int64_t width = t.shape[0];
    if (row < 0 || row >= t.shape[1] || count != width) return FORTAI_GGUF_INVALID;
    for (int64_t i = 0; i < width; ++i)
        values[i] = fortai_gguf_tensor_value(file, index, row * width + i);
    return FORTAI_GGUF_OK;
}

extern "C" int fortai_gguf_upload_q8(const fortai_gguf_file *file, int64_t index,
    fortai_cuda_q8_context *context, int64_t first_row, int64_t row_count,
    fortai_cuda_q8_weights **weights) {
    if (weights) *weights = nullptr;
    if (!file || !context || !weights || index < 0 ||
        index >= static_cast<int64_t>(file->tensors.size())) return FORTAI_GGUF_INVALID;
    const Tensor &t = file->tensors[static_cast<size_t>(index)];
    if (t.rank != 2 || t.type != FORTAI_GGML_TYPE_Q8_0) return FORTAI_GGUF_INVALID;
    const int64_t width = t.shape[0], rows = t.shape[1];
    if (first_row < 0 || first_row >= rows || row_count < 0) return FORTAI_GGUF_INVALID;
    if (row_count == 0) row_count = rows - first_row;
    if (row_count > rows - first_row || width > 0x7fffffff || row_count > 0x7fffffff)
        return FORTAI_GGUF_INVALID;
    const int64_t row_bytes = (width / 32) * 34;
    const uint8_t *bytes = file->base + file->data_start + t.file_offset + first_row * row_bytes;
    const int code = fortai_cuda_q8_weights_upload(context, bytes,
        static_cast<size_t>(row_count * row_bytes), static_cast<int>(row_count),
        static_cast<int>(width), weights);
    return code == 0 ? FORTAI_GGUF_OK : FORTAI_GGUF_UNSUPPORTED;
}
