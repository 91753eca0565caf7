/* Reader of the `.ninfer` v2 container, as far as the quantized linear path needs it: open and
 * validate a container, list its object directory, and turn an NVFP4 or trellis tensor into the
 * weight view the kernels take (b200q_nvfp4_weight, ignis_trellis_weight).
 *
 * reference: crates/artifact/src/lib.rs - the framing (:145-161), the closed registries of
 * formats and layouts (:176-320), the payload geometry of every layout (:421-660), the closed JSON
 * directory (:743-856), Reader::open's checks in their order (:1075-1170), content_hash
 * (:1204-1240); crates/artifact/src/binding.rs:75-102 (the NVFP4 view); the object names of the
 * 27B NVFP4 artifact: docs/formats/27b-nvfp4-work-tree.md section 4.2. The reference's reader is
 * Rust; this is the same checks and the same messages in C++ behind a C ABI, host code only (no
 * CUDA call: the caller copies payloads to the device with whatever it uses for that).
 *
 * The container: 8 bytes of magic "NINFER\0\2", a little-endian u64 `json_bytes`, that many bytes
 * of JSON ({"identity": {"model_id", "weights_id"}, "objects": [...]}; trailing spaces allowed),
 * zero padding to a multiple of 4096, then the payload section. An object's `offset` is relative
 * to the payload section; objects lie in directory order without overlap, tensors on 256-byte
 * boundaries (trellis records and row-interleaved tables on 4096), resources on any byte.
 *
 * Every function returns 0, or -1 with the reason in b200q_artifact_last_error() (thread-local).
 */
#ifndef B200Q_ARTIFACT_H_
#define B200Q_ARTIFACT_H_

#include <stdint.h>

#include "b200q_nvfp4.h"
#include "ignis_trellis_linear.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200q_artifact b200q_artifact; /* an open, validated container */

#define B200Q_ARTIFACT_TENSOR 1u
#define B200Q_ARTIFACT_RESOURCE 2u

/* Numeric formats, in the registry's order (lib.rs:176-199). */
enum {
  B200Q_FORMAT_NONE = 0, /* a resource */
  B200Q_FORMAT_BF16,
  B200Q_FORMAT_FP32,
  B200Q_FORMAT_I32,
  B200Q_FORMAT_Q4G64_F16S,
  B200Q_FORMAT_Q5G64_F16S,
  B200Q_FORMAT_Q6G64_F16S,
  B200Q_FORMAT_W8G32_F16S,
  B200Q_FORMAT_NVFP4,
  B200Q_FORMAT_FP8_E4M3FN_ROW_BF16S,
  B200Q_FORMAT_I64,
  B200Q_FORMAT_Q4G32_F16S,
  B200Q_FORMAT_TRELLIS_MUL1_K2,
  B200Q_FORMAT_TRELLIS_MUL1_K2P5,
  B200Q_FORMAT_TRELLIS_MUL1_K3,
  B200Q_FORMAT_TRELLIS_MUL1_K4,
  B200Q_FORMAT_TRELLIS_MUL1_K5,
  B200Q_FORMAT_TRELLIS_MUL1_K6
};

/* Storage layouts (lib.rs:261-275) and the one resource encoding (:301-303). */
enum {
  B200Q_LAYOUT_NONE = 0,
  B200Q_LAYOUT_CONTIGUOUS_LE_V1,
  B200Q_LAYOUT_ROW_SPLIT_K128_V1,
  B200Q_LAYOUT_BLOCKSCALE_K16_M128X4_V1,
  B200Q_LAYOUT_ROW_SCALE_V1,
  B200Q_LAYOUT_TRELLIS_TILE16_V1,
  B200Q_LAYOUT_ROW_INTERLEAVED_V1,
  B200Q_LAYOUT_RAW_BYTES_V1 /* resources */
};

#define B200Q_ARTIFACT_MAX_RANK 16

typedef struct b200q_artifact_object {
  const char *name;   /* lives as long as the artifact stays open */
  uint32_t kind;      /* B200Q_ARTIFACT_TENSOR or _RESOURCE */
  uint32_t format;    /* B200Q_FORMAT_* */
  uint32_t layout;    /* B200Q_LAYOUT_* */
  uint32_t rank;      /* 0 for a scalar and for a resource */
  uint64_t shape[B200Q_ARTIFACT_MAX_RANK]; /* outermost first */
  uint64_t offset;    /* relative to the payload section */
  uint64_t bytes;     /* exact stored length */
  uint64_t file_offset; /* absolute: payload section start + offset */
  const void *data;   /* the payload in this process's read-only mapping of the file */
} b200q_artifact_object;

/* Offsets inside one payload, relative to its first byte. reference: BlockScaleGeometry
 * (lib.rs:362-373, :597-634) and TrellisGeometry (:393-407, :498-524). */
typedef struct b200q_blockscale_geometry {
  uint64_t rows, columns, groups_per_row, k_tiles;
  uint64_t code_plane_bytes, scale_plane_offset, scale_plane_bytes, weight_divisor_offset, encoded_bytes;
} b200q_blockscale_geometry;

typedef struct b200q_trellis_geometry {
  uint64_t rows, columns, k2; /* shape [out, in] = [rows, columns] */
  uint64_t trellis_bytes, suh_offset, svh_offset, data_bytes, encoded_bytes;
} b200q_trellis_geometry;

/* ---- geometry (no file needed) ---- */

/* Registry lookups by the directory's spelling ("NVFP4", "blockscale-k16-m128x4-v1", ...):
 * the B200Q_FORMAT_ / B200Q_LAYOUT_ value, or 0 with the error set for an unknown name. */
uint32_t b200q_artifact_format_by_name(const char *name);
uint32_t b200q_artifact_layout_by_name(const char *name);
const char *b200q_artifact_format_name(uint32_t format); /* NULL for a value outside the registry */
const char *b200q_artifact_layout_name(uint32_t layout);
/* 2 K of a trellis format (4, 5, 6, 8, 10, 12), 0 for any other (lib.rs:228-238). */
uint32_t b200q_artifact_trellis_k2(uint32_t format);
/* File alignment of a layout's payloads: 256, or 4096 for trellis records and row-interleaved
 * tables; 1 for resources (lib.rs:323-336). */
uint64_t b200q_artifact_alignment(uint32_t layout);

/* Exact stored size of a tensor; what the directory's `bytes` must equal (lib.rs:456-492). */
int32_t b200q_artifact_encoded_size(uint32_t layout, uint32_t format, const uint64_t *shape, uint32_t rank,
                                    uint64_t *bytes);
int32_t b200q_artifact_blockscale_geometry(uint32_t format, const uint64_t *shape, uint32_t rank,
                                           b200q_blockscale_geometry *out);
int32_t b200q_artifact_trellis_geometry(uint32_t format, const uint64_t *shape, uint32_t rank,
                                        b200q_trellis_geometry *out);

/* ---- the container ---- */

/* Opens, maps and validates `path` (Reader::open, lib.rs:1075-1170): the prefix, the closed JSON
 * schema, every tensor's stored size against its layout, then order, alignment, bounds and
 * duplicate names. On success *out owns the mapping until b200q_artifact_close. */
int32_t b200q_artifact_open(const char *path, b200q_artifact **out);
void b200q_artifact_close(b200q_artifact *artifact);

const char *b200q_artifact_model_id(const b200q_artifact *artifact);
const char *b200q_artifact_weights_id(const b200q_artifact *artifact);
uint64_t b200q_artifact_object_count(const b200q_artifact *artifact);
uint64_t b200q_artifact_payload_offset(const b200q_artifact *artifact); /* 4096-aligned */
uint64_t b200q_artifact_file_bytes(const b200q_artifact *artifact);
int32_t b200q_artifact_object_at(const b200q_artifact *artifact, uint64_t index, b200q_artifact_object *out);
/* By exact name; -1 ("unknown artifact object: <name>") if the directory has none. */
int32_t b200q_artifact_find(const b200q_artifact *artifact, const char *name, b200q_artifact_object *out);
/* SHA-256 over what the directory declares (identity, sizes, every object's name, kind, offset,
 * length, format, layout, shape), not over the payload (Reader::content_hash, lib.rs:1204-1240). */
int32_t b200q_artifact_content_hash(const b200q_artifact *artifact, uint8_t digest[32]);

/* ---- weight views ---- */

/* The name of the rank-0 FP32 activation divisor that follows an NVFP4 projection of the 27B
 * artifact (work-tree section 4.2): <layer>/gdn/query_key_value_z -> <layer>/gdn/input_projection/
 * input_scale_divisor, gdn/output -> gdn/output_projection/..., attention/query_key_gate_value ->
 * attention/input_projection/..., attention/output -> attention/output_projection/...,
 * mlp/gate_up -> mlp/gate_up_projection/..., mlp/down -> mlp/down_projection/.... Writes the
 * NUL-terminated name into `out`; -1 if `parent` ends in none of the six or `capacity` is short. */
int32_t b200q_artifact_divisor_name(const char *parent, char *out, uint64_t capacity);

/* The view of NVFP4 tensor `name` for a copy of its payload at `payload` (device memory the caller
 * filled with the object's `bytes`, 256-byte aligned; NULL = the host mapping itself, for host-side
 * decoding). codes = payload, scales = payload + scale_plane_offset, the weight divisor is read
 * from the file. `divisor`: the name of its rank-0 FP32 activation divisor; NULL derives it with
 * b200q_artifact_divisor_name and requires it to exist; "" means the tensor has none (1.0).
 * Refuses a tensor that is not NVFP4 / blockscale-k16-m128x4-v1 / rank two, a divisor object of
 * another format or shape, and divisors that are not finite and positive. */
int32_t b200q_artifact_nvfp4_weight(const b200q_artifact *artifact, const char *name, const char *divisor,
                                    const void *payload, b200q_nvfp4_weight *out);

/* The view of trellis tensor `name` (shape [out, in]) for a copy of its record at `payload`
 * (device memory, 256-byte aligned; NULL = the host mapping): trellis = payload, suh = payload +
 * suh_offset (fp16 [in]), svh = payload + svh_offset (fp16 [out]), k2 from the format,
 * tile_stride 0. */
int32_t b200q_artifact_trellis_weight(const b200q_artifact *artifact, const char *name, const void *payload,
                                      ignis_trellis_weight *out);

const char *b200q_artifact_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_ARTIFACT_H_ */
