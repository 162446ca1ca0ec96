// Native GGUF tensor-table reader and per-tensor loader with a persisted repack.
//
// The reference reads the GGUF header in C# (src/Synapse.Runtime/Features/ModelLoading/Gguf/GgufHeaderReader.cs:20-154),
// maps the file (Gguf/GgufFile.cs:76-98) and its CUDA backend copies the WHOLE file to the device
// (native/synapse-gpu/src/Features/GpuKernels/cuda/decoder.rs:59-60). Here the native side parses the same header
// (GGUF v2 / v3: magic, version, tensor and metadata counts, metadata key/values, tensor infos, data section aligned to
// general.alignment, default 32) with the same bounds and failure rules, and uploads tensor by tensor straight from the
// mapping. A repacked (planar) device image can be written to a cache directory and is then read back instead of
// repacking again; cache entries are keyed by a digest of the file's header and length plus the tensor's place in it.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"

struct syn_b200_gguf {
    int fd = -1;
    const uint8_t *data = nullptr;
    uint64_t length = 0;
    uint32_t version = 0;
    uint64_t alignment = 32, data_offset = 0, digest = 0;
    std::vector<syn_b200_gguf_tensor> tensors;
    std::unordered_map<std::string, size_t> by_name;
};

namespace syn {
namespace {

constexpr uint32_t kMagic = 0x46554747u;  // "GGUF"
constexpr uint64_t kMaximumCount = 1000000, kMaximumArrayElements = 10000000;

struct Malformed {
    std::string message;
};

// A bounds-checked cursor over the mapped file.
struct Cursor {
    const uint8_t *data;
    uint64_t length, at = 0;
    void need(uint64_t bytes) const
    {
        if (bytes > length - at) {
            throw Malformed{"GGUF header is truncated."};
        }
    }
    template <class T>
    T read()
    {
        need(sizeof(T));
        T value;
        memcpy(&value, data + at, sizeof(T));
        at += sizeof(T);
        return value;
    }
    std::string read_string()
    {
        const uint64_t size = read<uint64_t>();
        if (size > (1u << 20)) {
            throw Malformed{"GGUF string of " + std::to_string(size) + " bytes exceeds the limit."};
        }
        need(size);
        std::string value(reinterpret_cast<const char *>(data + at), size);
        at += size;
        return value;
    }
    void skip(uint64_t bytes)
    {
        need(bytes);
        at += bytes;
    }
};

uint64_t bounded_count(Cursor &c, const char *what, uint64_t maximum)
{
    const uint64_t count = c.read<uint64_t>();
    if (count > maximum) {
        throw Malformed{std::string("GGUF ") + what + " count " + std::to_string(count) + " exceeds the limit."};
    }
    return count;
}

// Bytes of a fixed-size metadata value type, 0 for strings / arrays / unknown types.
uint64_t scalar_bytes(uint32_t type)
{
    switch (type) {
    case 0: case 1: case 7: return 1;   // u8, i8, bool
    case 2: case 3: return 2;           // u16, i16
    case 4: case 5: case 6: return 4;   // u32, i32, f32
    case 10: case 11: case 12: return 8;  // u64, i64, f64
    default: return 0;
    }
}

// Skips one metadata value; returns it as an integer when it is an integer scalar (for general.alignment).
bool skip_value(Cursor &c, uint32_t type, int depth, int64_t *integer)
{
    if (type == 8) {
        c.read_string();
        return false;
    }
    if (type == 9) {
        if (depth >= 4) {
            throw Malformed{"GGUF metadata arrays are nested too deeply."};
        }
        const uint32_t element = c.read<uint32_t>();
        const uint64_t count = bounded_count(c, "array element", kMaximumArrayElements);
        if (const uint64_t bytes = scalar_bytes(element)) {
            c.skip(bytes * count);
        } else {
            for (uint64_t i = 0; i < count; ++i) {
                skip_value(c, element, depth + 1, nullptr);
            }
        }
        return false;
    }
    const uint64_t bytes = scalar_bytes(type);
    if (bytes == 0) {
        throw Malformed{"GGUF metadata value type " + std::to_string(type) + " is unknown."};
    }
    bool is_integer = false;
    if (integer) {
        switch (type) {
        case 0: *integer = c.data[c.at]; is_integer = true; break;
        case 1: *integer = (int8_t)c.data[c.at]; is_integer = true; break;
        case 2: { uint16_t v; memcpy(&v, c.data + c.at, 2); *integer = v; is_integer = true; break; }
        case 3: { int16_t v; memcpy(&v, c.data + c.at, 2); *integer = v; is_integer = true; break; }
        case 4: { uint32_t v; memcpy(&v, c.data + c.at, 4); *integer = v; is_integer = true; break; }
        case 5: { int32_t v; memcpy(&v, c.data + c.at, 4); *integer = v; is_integer = true; break; }
        case 10: case 11: { int64_t v; memcpy(&v, c.data + c.at, 8); *integer = v; is_integer = true; break; }
        default: break;
        }
    }
    c.skip(bytes);
    return is_integer;
}

uint64_t fnv1a(const uint8_t *data, uint64_t size, uint64_t state = 0xcbf29ce484222325ull)
{
    for (uint64_t i = 0; i < size; ++i) {
        state = (state ^ data[i]) * 0x100000001b3ull;
    }
    return state;
}

// Parses the header; throws Malformed (status 2) or returns a status with the message recorded.
int32_t parse(syn_b200_gguf &g)
{
    Cursor c{g.data, g.length};
    if (c.read<uint32_t>() != kMagic) {
        throw Malformed{"The file is not a GGUF model."};
    }
    g.version = c.read<uint32_t>();
    if (g.version < 2 || g.version > 3) {
        throw Malformed{"GGUF version " + std::to_string(g.version) + " is not supported."};
    }
    const uint64_t tensor_count = bounded_count(c, "tensor", kMaximumCount);
    const uint64_t metadata_count = bounded_count(c, "metadata", kMaximumCount);
    for (uint64_t i = 0; i < metadata_count; ++i) {
        const std::string key = c.read_string();
        const uint32_t type = c.read<uint32_t>();
        int64_t integer = 0;
        if (skip_value(c, type, 0, &integer) && key == "general.alignment") {
            if (integer <= 0 || (integer & (integer - 1)) != 0) {
                throw Malformed{"GGUF alignment " + std::to_string(integer) + " is invalid."};
            }
            g.alignment = (uint64_t)integer;
        }
    }
    struct Header {
        std::string name;
        uint32_t rank, type;
        uint64_t dimensions[8], relative;
    };
    std::vector<Header> headers(tensor_count);
    for (Header &h : headers) {
        h.name = c.read_string();
        h.rank = c.read<uint32_t>();
        if (h.rank == 0 || h.rank > 8) {
            throw Malformed{"Tensor '" + h.name + "' has invalid rank " + std::to_string(h.rank) + "."};
        }
        for (uint32_t d = 0; d < 8; ++d) {
            h.dimensions[d] = d < h.rank ? c.read<uint64_t>() : 1;
        }
        h.type = c.read<uint32_t>();
        h.relative = c.read<uint64_t>();
    }
    g.data_offset = (c.at + g.alignment - 1) / g.alignment * g.alignment;
    g.digest = fnv1a(reinterpret_cast<const uint8_t *>(&g.length), sizeof(g.length), fnv1a(g.data, c.at));
    for (const Header &h : headers) {
        uint64_t elements = 1;
        for (uint32_t d = 0; d < h.rank; ++d) {
            if (h.dimensions[d] > (uint64_t)INT64_MAX || __builtin_mul_overflow(elements, h.dimensions[d], &elements) || elements > (uint64_t)INT64_MAX) {
                throw Malformed{"Tensor '" + h.name + "' overflows."};
            }
        }
        uint64_t bytes = 0;
        if (h.type == 0) {
            bytes = elements * 4;
        } else if (h.type == kQ8_0 && elements % 32 == 0) {
            bytes = elements / 32 * 34;
        } else if (h.type == kQ4_K && elements % 256 == 0) {
            bytes = elements / 256 * 144;
        } else if (h.type == kQ6_K && elements % 256 == 0) {
            bytes = elements / 256 * 210;
        } else {
            return fail(SYN_B200_UNAVAILABLE, "Tensor '" + h.name + "' uses unsupported GGML type " + std::to_string(h.type) + ".");
        }
        uint64_t absolute = 0;
        if (__builtin_add_overflow(g.data_offset, h.relative, &absolute) || absolute > g.length || bytes > g.length - absolute) {
            throw Malformed{"Tensor '" + h.name + "' is outside the GGUF file."};
        }
        syn_b200_gguf_tensor t{};
        snprintf(t.name, sizeof(t.name), "%s", h.name.c_str());
        t.ggml_type = h.type;
        t.rank = h.rank;
        memcpy(t.dimensions, h.dimensions, sizeof(t.dimensions));
        t.offset = absolute;
        t.bytes = bytes;
        g.by_name.emplace(h.name, g.tensors.size());
        g.tensors.push_back(t);
    }
    return SYN_B200_OK;
}

// ---- persisted device images of repacked matrices ---------------------------------------------------------

struct ImageHeader {
    char magic[8];  // "SYNB200M"
    uint32_t version, type, layout, flags;
    uint64_t rows, columns, row_bytes, planes[4], data_bytes, digest, tensor_offset, tensor_bytes;
};

std::string image_path(const syn_b200_gguf &g, const syn_b200_gguf_tensor &t, const char *directory)
{
    char name[64];
    snprintf(name, sizeof(name), "%016llx-%016llx.synb200", (unsigned long long)g.digest, (unsigned long long)fnv1a(reinterpret_cast<const uint8_t *>(t.name), strlen(t.name), t.offset));
    return std::string(directory) + "/" + name;
}

ImageHeader image_header(const syn_b200_gguf &g, const syn_b200_gguf_tensor &t, const syn_b200_matrix &m)
{
    ImageHeader h{};
    memcpy(h.magic, "SYNB200M", 8);
    h.version = 1;
    h.type = m.type;
    h.layout = (uint32_t)m.layout;
    h.flags = m.flags;
    h.rows = m.rows;
    h.columns = m.columns;
    h.row_bytes = m.row_bytes;
    h.planes[0] = m.planes.p0;
    h.planes[1] = m.planes.p1;
    h.planes[2] = m.planes.p2;
    h.planes[3] = m.planes.p3;
    h.data_bytes = m.data_bytes;
    h.digest = g.digest;
    h.tensor_offset = t.offset;
    h.tensor_bytes = t.bytes;
    return h;
}

// Reads a cached image into a new matrix; nullptr when there is none or it does not belong to this tensor.
syn_b200_matrix *load_image(const syn_b200_gguf &g, const syn_b200_gguf_tensor &t, uint32_t flags, const std::string &path, int device)
{
    FILE *file = fopen(path.c_str(), "rb");
    if (!file) {
        return nullptr;
    }
    ImageHeader h{};
    syn_b200_matrix *m = nullptr;
    std::vector<uint8_t> payload;
    if (fread(&h, sizeof(h), 1, file) == 1 && memcmp(h.magic, "SYNB200M", 8) == 0 && h.version == 1 && h.type == t.ggml_type && h.flags == flags &&
        h.rows == t.dimensions[1] && h.columns == t.dimensions[0] && h.digest == g.digest && h.tensor_offset == t.offset && h.tensor_bytes == t.bytes &&
        h.layout == (uint32_t)Layout::Planar && h.data_bytes < (1ull << 40)) {
        payload.resize(h.data_bytes);
        if (fread(payload.data(), 1, payload.size(), file) == payload.size()) {
            m = new syn_b200_matrix();
            m->type = h.type;
            m->flags = h.flags;
            m->rows = h.rows;
            m->columns = h.columns;
            m->row_bytes = h.row_bytes;
            m->device = device;
            m->layout = Layout::Planar;
            m->planes.p0 = h.planes[0];
            m->planes.p1 = h.planes[1];
            m->planes.p2 = h.planes[2];
            m->planes.p3 = h.planes[3];
            m->data_bytes = h.data_bytes;
            if (cudaMalloc(&m->data, m->data_bytes + 64) != cudaSuccess || cudaMemcpy(m->data, payload.data(), m->data_bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
                cudaGetLastError();
                if (m->data) {
                    cudaFree(m->data);
                }
                delete m;
                m = nullptr;
            }
        }
    }
    fclose(file);
    return m;
}

void save_image(const syn_b200_gguf &g, const syn_b200_gguf_tensor &t, const syn_b200_matrix &m, const std::string &path)
{
    std::vector<uint8_t> payload(m.data_bytes);
    if (cudaMemcpy(payload.data(), m.data, m.data_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    const std::string temporary = path + ".tmp" + std::to_string((long)getpid());
    FILE *file = fopen(temporary.c_str(), "wb");
    if (!file) {
        return;  // a cache that cannot be written is not an error
    }
    const ImageHeader h = image_header(g, t, m);
    const bool written = fwrite(&h, sizeof(h), 1, file) == 1 && fwrite(payload.data(), 1, payload.size(), file) == payload.size();
    if (fclose(file) == 0 && written) {
        rename(temporary.c_str(), path.c_str());
    } else {
        remove(temporary.c_str());
    }
}

}  // namespace
}  // namespace syn

using namespace syn;

extern "C" {

int32_t syn_b200_gguf_open(const char *path, syn_b200_gguf **out)
{
    if (!path || !out) {
        return fail(SYN_B200_NULL_POINTER, "path or output handle");
    }
    *out = nullptr;
    return guarded([&]() -> int32_t {
        const int fd = open(path, O_RDONLY);
        if (fd < 0) {
            return fail(SYN_B200_INVALID_ARGUMENT, std::string("cannot open '") + path + "'");
        }
        struct stat info {};
        if (fstat(fd, &info) != 0 || info.st_size < 24) {
            close(fd);
            return fail(SYN_B200_INVALID_ARGUMENT, "GGUF header is truncated.");
        }
        void *mapping = mmap(nullptr, (size_t)info.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
        if (mapping == MAP_FAILED) {
            close(fd);
            return fail(SYN_B200_INVALID_ARGUMENT, std::string("cannot map '") + path + "'");
        }
        syn_b200_gguf *g = new syn_b200_gguf();
        g->fd = fd;
        g->data = static_cast<const uint8_t *>(mapping);
        g->length = (uint64_t)info.st_size;
        int32_t status;
        try {
            status = parse(*g);
        } catch (const Malformed &problem) {
            status = fail(SYN_B200_INVALID_ARGUMENT, problem.message);
        }
        if (status != SYN_B200_OK) {
            syn_b200_gguf_close(g);
            return status;
        }
        *out = g;
        return SYN_B200_OK;
    });
}

void syn_b200_gguf_close(syn_b200_gguf *gguf)
{
    if (!gguf) {
        return;
    }
    if (gguf->data) {
        munmap(const_cast<uint8_t *>(gguf->data), (size_t)gguf->length);
    }
    if (gguf->fd >= 0) {
        close(gguf->fd);
    }
    delete gguf;
}

uint64_t syn_b200_gguf_tensor_count(const syn_b200_gguf *gguf) { return gguf ? gguf->tensors.size() : 0; }

int32_t syn_b200_gguf_tensor_at(const syn_b200_gguf *gguf, uint64_t index, syn_b200_gguf_tensor *out)
{
    if (!gguf || !out) {
        return fail(SYN_B200_NULL_POINTER, "file or output");
    }
    if (index >= gguf->tensors.size()) {
        return fail(SYN_B200_INVALID_ARGUMENT, "tensor index " + std::to_string(index) + " is outside the table of " + std::to_string(gguf->tensors.size()));
    }
    *out = gguf->tensors[index];
    return SYN_B200_OK;
}

int32_t syn_b200_gguf_find(const syn_b200_gguf *gguf, const char *name, syn_b200_gguf_tensor *out)
{
    if (!gguf || !name || !out) {
        return fail(SYN_B200_NULL_POINTER, "file, name or output");
    }
    return guarded([&]() -> int32_t {
        const auto found = gguf->by_name.find(name);
        if (found == gguf->by_name.end()) {
            return fail(SYN_B200_INVALID_ARGUMENT, std::string("the file has no tensor '") + name + "'");
        }
        *out = gguf->tensors[found->second];
        return SYN_B200_OK;
    });
}

const uint8_t *syn_b200_gguf_mapping(const syn_b200_gguf *gguf, uint64_t *length, uint64_t *data_offset)
{
    if (!gguf) {
        return nullptr;
    }
    if (length) {
        *length = gguf->length;
    }
    if (data_offset) {
        *data_offset = gguf->data_offset;
    }
    return gguf->data;
}

int32_t syn_b200_gguf_load_matrix(const syn_b200_gguf *gguf, const char *name, uint32_t flags, const char *cache_directory, syn_b200_matrix **out)
{
    if (!gguf || !name || !out) {
        return fail(SYN_B200_NULL_POINTER, "file, name or output handle");
    }
    *out = nullptr;
    return guarded([&]() -> int32_t {
        syn_b200_gguf_tensor t{};
        int32_t status = syn_b200_gguf_find(gguf, name, &t);
        if (status != SYN_B200_OK) {
            return status;
        }
        if (t.rank != 2 || block_values(t.ggml_type) == 0) {
            return fail(SYN_B200_INVALID_ARGUMENT, std::string("tensor '") + name + "' is not a two-dimensional Q8_0 / Q4_K / Q6_K matrix");
        }
        // GGUF stores the row length first: dimensions[0] = columns, dimensions[1] = rows (Q8Matrix.cs:51-54)
        const uint64_t columns = t.dimensions[0], rows = t.dimensions[1];
        const bool planar = (flags & SYN_B200_REPACK) && t.ggml_type != kQ4_K;
        std::string cached;
        if (cache_directory && planar) {
            cached = image_path(*gguf, t, cache_directory);
            int device = 0;
            if (cudaGetDevice(&device) == cudaSuccess) {
                if (syn_b200_matrix *m = load_image(*gguf, t, flags, cached, device)) {
                    *out = m;
                    return SYN_B200_OK;
                }
            }
            cudaGetLastError();
        }
        status = syn_b200_matrix_create(gguf->data + t.offset, t.ggml_type, rows, columns, flags, out);
        if (status == SYN_B200_OK && !cached.empty()) {
            save_image(*gguf, t, **out, cached);
        }
        return status;
    });
}

}  // extern "C"
