/* aotx_gguf_b200 - the model-file side of the Q8_0 path: find a tensor in a GGUF file and
 * put its rows, or one rank's share of its rows, into device memory in the layout the
 * kernels of aotx_q8_b200.h read.
 *
 * The kernels read the model file's block layout unchanged, so "loading" is a byte copy:
 * a row range [first, first + rows) of a tensor is the contiguous byte range
 * [first * row_bytes, (first + rows) * row_bytes) of its bytes, which is also exactly one
 * rank's shard of a column-split projection, and an expert range of a stacked expert tensor
 * is a row range of its outermost dimension.
 *
 * What this replaces in the reference (paths relative to its source root):
 *   disk/modelfile/modelfile.h:99-162    the reader's interface (open, tensor table, metadata
 *                                        getters, bounded reads)
 *   disk/modelfile/gguf.c, meta.c        its implementation
 *   cuda/boot/weights_host.cu:84-111     the two-buffer pinned upload of one tensor
 * The checks at open are the reference's (same refusals, same return codes), so a file that
 * one reader takes the other takes too; tests/test_gguf.py holds that comparison.
 *
 * Return codes of the reader follow the reference: 0 success, 1 the file cannot be read (or
 * a bad argument), 2 the format is wrong.  Metadata getters: 0 found, 1 no such key, 2 the
 * key holds another type.
 */
#ifndef AOTX_GGUF_B200_H
#define AOTX_GGUF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AOTX_GGUF_OK 0
#define AOTX_GGUF_ERR_READ 1
#define AOTX_GGUF_ERR_FORMAT 2
#define AOTX_GGUF_ERR_CUDA 3 /* upload only: a CUDA call failed; see aotx_gguf_loader_last_cuda_error */

#define AOTX_GGUF_NAME_BYTES 128u
#define AOTX_GGUF_DIMS 4u

/* One row of the tensor table.  Same fields, order and sizes as the reference's
 * aotx_tensor_info (disk/modelfile/modelfile.h:99-106), so either struct can be passed
 * where the other is expected.  dims[0] is the row length (the fastest dimension); unused
 * dimensions read 1.  `bytes` is 0 for a block type this reader has no layout for. */
typedef struct aotx_gguf_tensor_info {
    char name[AOTX_GGUF_NAME_BYTES];
    uint32_t dim_count;
    uint32_t type;
    uint64_t dims[AOTX_GGUF_DIMS];
    uint64_t offset; /* from the start of the tensor bytes */
    uint64_t bytes;
} aotx_gguf_tensor_info;

typedef struct aotx_gguf aotx_gguf;

/* Open a file, check the header, the metadata and the tensor table (version 3; alignment from
 * general.alignment or 32; every tensor inside the tensor bytes and on the alignment; names and
 * keys unique).  Replaces aotx_modelfile_open / close (disk/modelfile/modelfile.h:118-125). */
int aotx_gguf_open(const char *path, aotx_gguf **file);
void aotx_gguf_close(aotx_gguf *file);

/* Sizes of the open file: all of it, the part before the tensor bytes (header, metadata,
 * tensor table, without the padding), and the tensor bytes
 * (disk/modelfile/modelfile.h:135-136,157). */
uint64_t aotx_gguf_file_bytes(const aotx_gguf *file);
uint64_t aotx_gguf_header_bytes(const aotx_gguf *file);
uint64_t aotx_gguf_data_bytes(const aotx_gguf *file);
uint32_t aotx_gguf_alignment(const aotx_gguf *file);

/* The tensor table (disk/modelfile/modelfile.h:153-156). */
uint64_t aotx_gguf_tensor_count(const aotx_gguf *file);
int aotx_gguf_tensor(const aotx_gguf *file, uint64_t index, aotx_gguf_tensor_info *info);
int aotx_gguf_find(const aotx_gguf *file, const char *name, aotx_gguf_tensor_info *info);

/* Scalar and string metadata by key (disk/modelfile/modelfile.h:138-143).  Any whole-number
 * type that is not negative reads as u64 / u32 (u32 refuses values above 2^32 - 1); F32 and
 * F64 read as f32.  Arrays are checked at open and can be sized with aotx_gguf_array; their
 * elements come through the getters further down. */
int aotx_gguf_u32(const aotx_gguf *file, const char *key, uint32_t *value);
int aotx_gguf_u64(const aotx_gguf *file, const char *key, uint64_t *value);
int aotx_gguf_f32(const aotx_gguf *file, const char *key, float *value);
int aotx_gguf_string(const aotx_gguf *file, const char *key, const char **value, size_t *length);
int aotx_gguf_array(const aotx_gguf *file, const char *key, uint32_t *element_type, uint64_t *count);

/* Array values by key (disk/modelfile/modelfile.h:144-151), read from the file the first time
 * they are asked for and kept until close.  i32s gives arrays of I32 and of U32 whose elements
 * all fit int32; f32s arrays of F32; bools arrays of BOOL; strings arrays of STRING as one byte
 * run with count + 1 offsets (same layout as the reference's aotx_string_array,
 * disk/modelfile/modelfile.h:108-114).  The pointers stay valid until aotx_gguf_close. */
typedef struct aotx_gguf_string_array {
    uint64_t count;
    const uint8_t *bytes;    /* every string, one after the other, no separators */
    const uint64_t *offsets; /* string i is [offsets[i], offsets[i + 1]) */
} aotx_gguf_string_array;
int aotx_gguf_i32s(const aotx_gguf *file, const char *key, const int32_t **values, uint64_t *count);
int aotx_gguf_f32s(const aotx_gguf *file, const char *key, const float **values, uint64_t *count);
int aotx_gguf_bools(const aotx_gguf *file, const char *key, const uint8_t **values, uint64_t *count);
int aotx_gguf_strings(const aotx_gguf *file, const char *key, aotx_gguf_string_array *array);

/* Read tensor bytes into host memory; offset from the start of the tensor bytes
 * (disk/modelfile/modelfile.h:159-162). */
int aotx_gguf_read(const aotx_gguf *file, uint64_t offset, uint64_t bytes, void *buffer);

/* The same read split over up to `threads` host threads (slices of at least 4 MiB, cut on
 * 4 KiB boundaries); one thread of a host reads a page-cached or NVMe-backed file well below
 * the rate a B200's link takes.  The upload below reads its pieces this way.  No counterpart
 * in the reference, whose loader reads on one thread. */
int aotx_gguf_read_threads(const aotx_gguf *file, uint64_t offset, uint64_t bytes, void *buffer,
                           uint32_t threads);

/* Bytes per row (dims[0] weights) of a block type, 0 for a type without a layout here or a
 * row that is not a whole number of blocks.  No counterpart as a function in the reference
 * (it is the arithmetic of disk/modelfile/gguf.c:158-194). */
uint64_t aotx_gguf_row_bytes(uint32_t type, uint64_t row_weights);

/* The byte range, inside the tensor bytes, of rows [first_row, first_row + rows) of a tensor,
 * counting rows over all dimensions above the first (a [k][n] matrix has n rows, a stacked
 * expert tensor [k][n][experts] has n * experts).  Returns 1 when the range leaves the tensor
 * or the type has no layout.  No counterpart in the reference, which loads whole tensors. */
int aotx_gguf_row_range(const aotx_gguf_tensor_info *info, uint64_t first_row, uint64_t rows,
                        uint64_t *offset, uint64_t *bytes);

/* Upload.  A loader owns two pinned host buffers of `piece_bytes` each (0 = 64 MiB, the
 * reference's size) and two events; the disk read of one piece overlaps the copy of the
 * piece before it.  Make it once, outside stream capture.  One loader serves one upload at a
 * time.  Replaces aotx_model_weights_open / close (cuda/boot/weights_host.cu:53-82). */
typedef struct aotx_gguf_loader aotx_gguf_loader;
int aotx_gguf_loader_init(aotx_gguf_loader **loader, int device, size_t piece_bytes);
int aotx_gguf_loader_destroy(aotx_gguf_loader *loader);
int aotx_gguf_loader_last_cuda_error(const aotx_gguf_loader *loader);

/* Copy [offset, offset + bytes) of the tensor bytes to device_dst, enqueued on `stream` in
 * pieces; returns when the last piece has been read from the file and its copy enqueued (the
 * copies themselves complete in stream order; synchronise the stream before the first use).
 * Replaces aotx_weights_stream (cuda/boot/weights_host.cu:84-111). */
int aotx_gguf_upload(aotx_gguf_loader *loader, const aotx_gguf *file, uint64_t offset, uint64_t bytes,
                     void *device_dst, void *stream);

/* The same for `rows` rows of `row_bytes` bytes each that lie back to back in the file from
 * `offset` and land `dst_pitch` bytes apart on the device (dst_pitch >= row_bytes).  Two calls
 * with dst_pitch = 2 * row_bytes, the second starting row_bytes further, interleave the rows of
 * a gate and an up tensor: the layout AOTX_Q8_EPILOGUE_SWIGLU and aotx_q8_moe_ffn_fused read
 * (include/aotx_q8_b200.h).  A piece holds whole rows; row_bytes above the loader's piece size
 * returns 1.  No counterpart in the reference. */
int aotx_gguf_upload_rows(aotx_gguf_loader *loader, const aotx_gguf *file, uint64_t offset,
                          uint64_t row_bytes, uint64_t rows, void *device_dst, uint64_t dst_pitch,
                          void *stream);

#ifdef __cplusplus
}
#endif

#endif
