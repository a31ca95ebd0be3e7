/*
 * llamd_gguf.h -- C ABI of the GGUF reader and the file-backed model loader in libllamd_cuda.so.
 *
 * The counterpart of the reference's file path into the device model:
 *   Gguf::open / parse / tensor / tensor_data     crates/llamd-gguf/src/lib.rs:116-286
 *   Hparams::from_gguf / validate                 crates/llamd-models/src/hparams.rs:78-186
 *   LayerNames::new, Model::open, verify_present  crates/llamd-models/src/model.rs:43-160
 *   DeviceModel::load_batched (upload order, the refusals before the upload)
 *                                                 crates/llamd-runtime/src/device.rs:225-471
 *
 * The file is mapped read-only and tensors go from the mapping to the device without an intermediate copy of the
 * model in host memory. Functions that can fail return one of the LLAMD_E_* kinds (the variants of
 * llamd_core::Error, crates/llamd-core/src/lib.rs:18-43) and write a message into `err` (may be NULL).
 */
#ifndef LLAMD_GGUF_H
#define LLAMD_GGUF_H

#include <stddef.h>
#include <stdint.h>

#include "llamd_cuda_model.h"

#ifdef __cplusplus
extern "C" {
#endif

enum {
    LLAMD_E_OK = 0,
    LLAMD_E_MALFORMED = -1,   /* Error::Malformed: the file contradicts the format or itself */
    LLAMD_E_UNSUPPORTED = -2, /* Error::Unsupported: valid, but not implemented (version, type, architecture) */
    LLAMD_E_IO = -3,          /* Error::Io: open / stat / mmap failed */
    LLAMD_E_OTHER = -4,       /* Error::Other: device-side failure during the upload, not enough memory */
    LLAMD_E_ABSENT = -5       /* a key or tensor that is simply not there (Option::None in the reference) */
};

/* ggml type ids the reader knows (QuantType, crates/llamd-quant/src/lib.rs:47-69) */
enum { LLAMD_GGML_F32 = 0, LLAMD_GGML_F16 = 1, LLAMD_GGML_Q8_0 = 8, LLAMD_GGML_Q6_K = 14 };

typedef struct llamd_gguf llamd_gguf;

/* Gguf::open (lib.rs:116-122): map the file and parse header, metadata and tensor table. NULL on failure with
 * *kind and err set. */
llamd_gguf *llamd_gguf_open(const char *path, int *kind, char *err, size_t err_len);
/* The same parse over caller-owned bytes, which must outlive the handle (Gguf::parse, lib.rs:124-213). */
llamd_gguf *llamd_gguf_parse(const void *bytes, size_t len, int *kind, char *err, size_t err_len);
void llamd_gguf_close(llamd_gguf *g);

uint32_t llamd_gguf_version(const llamd_gguf *g);
uint64_t llamd_gguf_alignment(const llamd_gguf *g);   /* general.alignment, default 32 (lib.rs:20,181-190) */
uint64_t llamd_gguf_data_offset(const llamd_gguf *g); /* first byte of the tensor data section (lib.rs:192-202) */
uint64_t llamd_gguf_file_size(const llamd_gguf *g);
uint64_t llamd_gguf_n_metadata(const llamd_gguf *g);
uint64_t llamd_gguf_n_tensors(const llamd_gguf *g);

/* Metadata lookups with the reference's conversions (Value::as_u64 / as_f32 / as_str / as_array, lib.rs:42-81):
 * as_u64 takes any unsigned type and non-negative signed ones; as_f32 takes F32 and F64. LLAMD_E_OK, or
 * LLAMD_E_ABSENT when the key is missing or of another type. get_str copies at most len-1 bytes and terminates;
 * *full_len (may be NULL) gets the string's length. */
int llamd_gguf_get_u64(const llamd_gguf *g, const char *key, uint64_t *out);
int llamd_gguf_get_f32(const llamd_gguf *g, const char *key, float *out);
int llamd_gguf_get_str(const llamd_gguf *g, const char *key, char *out, size_t len, size_t *full_len);
int llamd_gguf_get_array_len(const llamd_gguf *g, const char *key, uint64_t *out);
/* Key of the i-th metadata entry in sorted order (the reference keeps a BTreeMap, lib.rs:107), NULL past the end. */
const char *llamd_gguf_metadata_key(const llamd_gguf *g, uint64_t i);

/* Tensor table (TensorInfo, lib.rs:88-102). find returns the index or -1 (Gguf::tensor, lib.rs:223-225: first match
 * in file order). */
int64_t llamd_gguf_find_tensor(const llamd_gguf *g, const char *name);
const char *llamd_gguf_tensor_name(const llamd_gguf *g, uint64_t index);
int llamd_gguf_tensor_info(const llamd_gguf *g, uint64_t index, uint32_t *ggml_type, int *n_dims, uint64_t dims[4],
                           uint64_t *offset);
/* Gguf::tensor_data (lib.rs:231-256): the tensor's bytes inside the mapping after the type, length
 * (QuantType::bytes_for refuses partial blocks) and extent checks. */
int llamd_gguf_tensor_data(const llamd_gguf *g, uint64_t index, const void **data, size_t *n_bytes, char *err,
                           size_t err_len);

/* Hparams::from_gguf + validate (hparams.rs:78-186). *is_moe (may be NULL) says which architecture key was read
 * ("qwen3moe" 1, "qwen3" 0); *n_ff and *n_ctx_train (may be NULL) get the two fields llamd_hparams does not carry. */
int llamd_gguf_hparams(const llamd_gguf *g, llamd_hparams *hp, int *is_moe, int32_t *n_ff, int32_t *n_ctx_train,
                       char *err, size_t err_len);
/* Model::verify_present (model.rs:133-160): every tensor the architecture needs exists. On failure the message
 * gives the count and the first three names. */
int llamd_gguf_verify_present(const llamd_gguf *g, char *err, size_t err_len);

/* DeviceModel::load_batched over an open file (device.rs:270-471): refuses dense models, a matrix
 * that is not Q6_K or not the shape the hyperparameters give it, and a model larger than free device memory, before
 * anything is uploaded (a file without output.weight loads with the head tied to the embedding table); then creates the
 * resident model and uploads every tensor from the mapping. With expert parallelism initialised, a rank reads
 * only its own experts' byte range of the three expert tensors. NULL on failure. */
llamd_model *llamd_model_load_gguf(const llamd_gguf *g, int max_kv, int max_seq, int *kind, char *err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif /* LLAMD_GGUF_H */
