// Native reader of the reference's `.bin` checkpoint container (host code only; it lives in this library so that a
// loader written in C++ needs nothing but libw8a8.so and include/w8a8_container.h).
//
// The format is src/model/tensor.h:53-67; what the reference's ModelLoader does with it is
// src/model/loader.cc:50-205: map the file, check magic and version, copy the headers into a name -> header table,
// hand out views by name. This reader does the same through mmap, and additionally refuses, at open, any header that
// the reference would follow blindly: unknown element type, more than eight dimensions, negative extents, a byte
// count that is not elements x element size, data that is not 256-byte aligned or that ends beyond the file.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/w8a8_container.h"
#include "w8a8_internal.h"

namespace {

constexpr uint32_t kMagic = 0x46495348u;  // "FISH", tensor.h:66
constexpr uint32_t kFormatVersion = 1;    // tensor.h:67
constexpr size_t kHeaderBytes = 344;      // tensor.h:55-64
constexpr uint64_t kAlign = 256;

struct Entry {
    std::string name;
    uint32_t dtype, ndim;
    int64_t shape[8];
    uint64_t offset, nbytes;
};

int element_size(uint32_t dtype) {  // dtype_size, tensor.h:15-23
    switch (dtype) {
        case W8A8_DTYPE_FP32: return 4;
        case W8A8_DTYPE_FP16: return 2;
        case W8A8_DTYPE_BF16: return 2;
        case W8A8_DTYPE_INT8: return 1;
        default: return 0;
    }
}

}  // namespace

struct w8a8_container {
    void* map = MAP_FAILED;
    size_t size = 0;
    bool pinned = false;
    std::vector<Entry> entries;
    std::unordered_map<std::string, int> by_name;
    uint64_t data_section_offset = 0;
};

using w8a8::fail;

extern "C" {

int w8a8_container_close(w8a8_container* c) {
    if (!c) return W8A8_OK;
    if (c->map != MAP_FAILED) {
        if (c->pinned) cudaHostUnregister(c->map);
        munmap(c->map, c->size);
    }
    delete c;
    return W8A8_OK;
}

int w8a8_container_open(const char* path, w8a8_container** out) {
    if (!path || !out) return fail(W8A8_ERR_INVALID_ARG, "w8a8_container_open: null argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(W8A8_ERR_INVALID_ARG, "Failed to open model file: %s (%s)", path, std::strerror(errno));
    struct stat st;
    if (fstat(fd, &st) < 0) {
        close(fd);
        return fail(W8A8_ERR_INVALID_ARG, "Failed to stat model file: %s", path);
    }
    w8a8_container* c = new w8a8_container;
    c->size = static_cast<size_t>(st.st_size);
    if (c->size < 12) {
        close(fd);
        delete c;
        return fail(W8A8_ERR_INVALID_ARG, "%s: shorter than the 12-byte preamble", path);
    }
    c->map = mmap(nullptr, c->size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);  // the mapping keeps the file
    if (c->map == MAP_FAILED) {
        delete c;
        return fail(W8A8_ERR_INVALID_ARG, "Failed to mmap model file: %s", path);
    }
    const unsigned char* p = static_cast<const unsigned char*>(c->map);
    uint32_t magic, version, count;
    std::memcpy(&magic, p, 4);
    std::memcpy(&version, p + 4, 4);
    std::memcpy(&count, p + 8, 4);
    auto refuse = [&](int rc) {
        w8a8_container_close(c);
        return rc;
    };
    if (magic != kMagic) return refuse(fail(W8A8_ERR_INVALID_ARG, "Invalid magic: 0x%08X, expected 0x%08X", magic, kMagic));
    if (version != kFormatVersion) return refuse(fail(W8A8_ERR_INVALID_ARG, "Unsupported version: %u", version));
    if (12 + static_cast<uint64_t>(count) * kHeaderBytes > c->size)
        return refuse(fail(W8A8_ERR_INVALID_ARG, "%s: %u headers do not fit in %zu bytes", path, count, c->size));
    c->entries.reserve(count);
    for (uint32_t i = 0; i < count; ++i) {
        const unsigned char* h = p + 12 + static_cast<size_t>(i) * kHeaderBytes;
        Entry e;
        e.name.assign(reinterpret_cast<const char*>(h), strnlen(reinterpret_cast<const char*>(h), 256));
        std::memcpy(&e.dtype, h + 256, 4);
        std::memcpy(&e.ndim, h + 260, 4);
        std::memcpy(e.shape, h + 264, 64);
        std::memcpy(&e.offset, h + 328, 8);
        std::memcpy(&e.nbytes, h + 336, 8);
        const int esz = element_size(e.dtype);
        if (!esz) return refuse(fail(W8A8_ERR_INVALID_ARG, "%s: unknown dtype %u", e.name.c_str(), e.dtype));
        if (e.ndim > 8) return refuse(fail(W8A8_ERR_INVALID_ARG, "%s: %u dimensions", e.name.c_str(), e.ndim));
        unsigned __int128 numel = 1;  // eight extents of up to 2^63 overflow 64 bits long before they describe a file
        for (uint32_t d = 0; d < e.ndim; ++d) {
            if (e.shape[d] < 0) return refuse(fail(W8A8_ERR_INVALID_ARG, "%s: negative extent", e.name.c_str()));
            numel *= static_cast<uint64_t>(e.shape[d]);
            if (numel > (static_cast<unsigned __int128>(1) << 62))
                return refuse(fail(W8A8_ERR_INVALID_ARG, "%s: extents overflow", e.name.c_str()));
        }
        for (uint32_t d = e.ndim; d < 8; ++d) e.shape[d] = 0;
        if (static_cast<unsigned __int128>(e.nbytes) != numel * static_cast<unsigned>(esz))
            return refuse(fail(W8A8_ERR_INVALID_ARG, "%s: %llu bytes do not match its shape", e.name.c_str(),
                               static_cast<unsigned long long>(e.nbytes)));
        if (e.offset % kAlign || e.offset > c->size || e.nbytes > c->size - e.offset)
            return refuse(fail(W8A8_ERR_INVALID_ARG, "%s: data at %llu+%llu is unaligned or outside the file", e.name.c_str(),
                               static_cast<unsigned long long>(e.offset), static_cast<unsigned long long>(e.nbytes)));
        c->by_name[e.name] = static_cast<int>(i);  // a repeated name: the later header wins, as in the reference's map
        c->entries.push_back(std::move(e));
    }
    c->data_section_offset = 12 + static_cast<uint64_t>(count) * kHeaderBytes;
    *out = c;
    return W8A8_OK;
}

int w8a8_container_count(const w8a8_container* c) { return c ? static_cast<int>(c->entries.size()) : 0; }

uint64_t w8a8_container_data_section_offset(const w8a8_container* c) { return c ? c->data_section_offset : 0; }

int w8a8_container_tensor(const w8a8_container* c, int index, w8a8_tensor_info* out) {
    if (!c || !out) return fail(W8A8_ERR_INVALID_ARG, "w8a8_container_tensor: null argument");
    if (index < 0 || index >= static_cast<int>(c->entries.size()))
        return fail(W8A8_ERR_INVALID_ARG, "w8a8_container_tensor: index %d of %zu", index, c->entries.size());
    const Entry& e = c->entries[index];
    out->name = e.name.c_str();
    out->dtype = static_cast<int>(e.dtype);
    out->ndim = static_cast<int>(e.ndim);
    std::memcpy(out->shape, e.shape, sizeof e.shape);
    out->offset = e.offset;
    out->nbytes = e.nbytes;
    out->data = static_cast<const unsigned char*>(c->map) + e.offset;
    return W8A8_OK;
}

int w8a8_container_find(const w8a8_container* c, const char* name) {
    if (!c || !name) return -1;
    auto it = c->by_name.find(name);
    if (it == c->by_name.end()) {
        fail(W8A8_ERR_INVALID_ARG, "Tensor not found: %s", name);
        return -1;
    }
    return it->second;
}

int w8a8_container_group_size(const w8a8_container* c, const char* weight, int* group_size) {
    if (!c || !weight || !group_size) return fail(W8A8_ERR_INVALID_ARG, "w8a8_container_group_size: null argument");
    const int wi = w8a8_container_find(c, weight);
    if (wi < 0) return W8A8_ERR_INVALID_ARG;
    const Entry& w = c->entries[wi];
    auto si = c->by_name.find(std::string(weight) + "_scale");
    if (w.dtype != W8A8_DTYPE_INT8 || si == c->by_name.end())
        return fail(W8A8_ERR_INVALID_ARG, "%s is not an int8 tensor with a _scale", weight);
    const Entry& s = c->entries[si->second];
    int64_t K = 1;  // infer_group_size_from_scale, dual_ar_engine.cc:17-24
    for (uint32_t d = 1; d < w.ndim; ++d) K *= w.shape[d];
    int64_t g = K;
    if (s.ndim > 1 && s.shape[1] > 1) g = (K + s.shape[1] - 1) / s.shape[1];
    *group_size = static_cast<int>(g);
    return W8A8_OK;
}

int w8a8_container_pin(w8a8_container* c) {
    if (!c || c->map == MAP_FAILED) return fail(W8A8_ERR_INVALID_ARG, "pin_memory: no mapped data");
    if (c->pinned) return W8A8_OK;
    const cudaError_t e = cudaHostRegister(c->map, c->size, cudaHostRegisterReadOnly);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(W8A8_ERR_CUDA, "pin_memory failed: %s (%zu MB)", cudaGetErrorString(e), c->size >> 20);
    }
    c->pinned = true;
    return W8A8_OK;
}

}  // extern "C"
