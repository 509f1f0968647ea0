/*
 * w8a8_container.h — C ABI of the native reader for the reference's `.bin` checkpoint container
 * (and for the packed sidecar this library writes in the same format).
 *
 * Replaces, for a host that loads the W8A8 linears of this library, the header pass and the
 * look-ups of fish::ModelLoader (src/model/loader.cc:50-171) over the file format of
 * src/model/tensor.h:53-67: magic "FISH" (u32 0x46495348), format version 1 (u32), tensor count
 * (u32), one 344-byte header per tensor {name[256], dtype u32, ndim u32, shape i64[8], data offset
 * u64, data size u64}, zero padding to a multiple of 256, tensor data at 256-byte aligned offsets.
 *
 * All pointers here are HOST pointers. The file is mapped read-only; tensor data is never
 * copied. Unlike the reference's loader, every header is checked against the file before it is
 * handed out (dtype known, ndim <= 8, extents non-negative, size = elements x element size, data
 * 256-byte aligned and inside the file): a file that points outside itself is refused at open.
 * Status codes and w8a8_last_error() as in w8a8.h.
 */
#ifndef W8A8_CONTAINER_H
#define W8A8_CONTAINER_H

#include "w8a8.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { /* DType values of src/model/tensor.h:8-13 */
    W8A8_DTYPE_FP32 = 0,
    W8A8_DTYPE_FP16 = 1,
    W8A8_DTYPE_BF16 = 2,
    W8A8_DTYPE_INT8 = 3
};

typedef struct w8a8_container w8a8_container;

typedef struct w8a8_tensor_info {
    const char* name;  /* owned by the container, valid until w8a8_container_close */
    int dtype;         /* W8A8_DTYPE_* */
    int ndim;
    int64_t shape[8];  /* extents beyond ndim are 0 */
    uint64_t offset;   /* of the data from the start of the file */
    uint64_t nbytes;
    const void* data;  /* inside the read-only mapping */
} w8a8_tensor_info;

/* Maps `path` and parses its headers: ModelLoader::load, src/model/loader.cc:50-153 (same refusals:
 * wrong magic, unsupported version; plus the bounds checks named above). W8A8_ERR_INVALID_ARG for a
 * file that is refused, W8A8_ERR_CUDA is never returned here (no device is touched). */
W8A8_API int w8a8_container_open(const char* path, w8a8_container** out);
/* ModelLoader::unload, src/model/loader.cc:189-205 (unpins first when pinned). */
W8A8_API int w8a8_container_close(w8a8_container* c);
W8A8_API int w8a8_container_count(const w8a8_container* c);
/* First byte after the headers (ModelLoader::data_section_offset_, loader.cc:150). */
W8A8_API uint64_t w8a8_container_data_section_offset(const w8a8_container* c);
/* Tensor number `index` in file order. */
W8A8_API int w8a8_container_tensor(const w8a8_container* c, int index, w8a8_tensor_info* out);
/* Index of the tensor called `name`, or -1: ModelLoader::has / get, src/model/loader.cc:155-171
 * (get's "Tensor not found: <name>" is left in w8a8_last_error()). */
W8A8_API int w8a8_container_find(const w8a8_container* c, const char* name);
/* Quantisation group size of the int8 tensor `weight`, from the shape of `<weight>_scale`:
 * infer_group_size_from_scale, src/engine/dual_ar_engine.cc:17-24 (K for a per-channel scale, else
 * ceil(K / groups) with K the product of the weight's extents after the first).
 * W8A8_ERR_INVALID_ARG when `weight` is not int8 or has no `_scale` (then it is not a W8A8 linear:
 * src/engine/dual_ar_engine.cc:240-249). */
W8A8_API int w8a8_container_group_size(const w8a8_container* c, const char* weight, int* group_size);
/* Page-locks the mapping for direct uploads: ModelLoader::pin_memory, src/model/loader.cc:173-187
 * (cudaHostRegister, read-only). W8A8_ERR_CUDA when the registration fails (no device, no memory). */
W8A8_API int w8a8_container_pin(w8a8_container* c);

#ifdef __cplusplus
}
#endif
#endif /* W8A8_CONTAINER_H */
