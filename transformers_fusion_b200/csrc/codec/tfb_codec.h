// libtfb_codec: the ".quant" ("QUA1") checkpoint container, its side-car index, SHA-256, the
// quantisation-format registry (105 formats) and the block codec.
//
// Wire compatibility with the reference project (include/quant/quant_format.h:15-34,
// src/codec/quant_format.cpp, src/codec/block_codec.cpp):
//   container   header | config | u32 n_fmt | {u32 id, u8 fmt, u32 cb}* | u32 n_tensors |
//               {u16 len, name, u32 start, u32 count}* | blocks {u32 nw, u32 cb, cb, u32 idx, idx}*
//   block streams: all 105 formats decode streams of the reference encoder bit-identically and encode streams of the
//   same layout and length (raw / truncated floats, lattice Q_8 / Q_4 / Q_2, fixed quantile codebooks, grouped affine,
//   6-bit scaled integers, compound 8 / 12-bit, four-tier mixes, the small-group fallback of short blocks).  A stream's
//   length follows from its layout; at ragged block sizes it can exceed ceil(bpw * n / 8) by a header byte, which
//   tfb_block_claimed_bytes accounts for.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TFB_FORMAT_COUNT 105
#define TFB_FMT_Q32 9
// Container header flag set by this library's writer when a file holds blocks of a format whose stream is this library's
// own encoding (tfb_format_is_wire_exact == 0).  Readers refuse such formats in files without the flag: those were written
// by another encoder with a different stream layout.
#define TFB_FLAG_OWN_STREAMS 0x40000000u

// ---- registry -------------------------------------------------------------------------------
const char* tfb_format_name(int fmt);            // "Q_4", "Q_G_8_K_M", ...; null when out of range
int tfb_format_parse(const char* name);          // accepts canonical names and legacy aliases (q4, qg8, Q4_K_M ...); -1 unknown
double tfb_format_bpw(int fmt);                  // claimed bits per weight
int tfb_format_is_grouped(int fmt);
int tfb_format_is_mix(int fmt);
int tfb_format_k_tier(int fmt);                  // 0 none, 1 L, 2 M, 3 H
int tfb_format_is_wire_exact(int fmt);
size_t tfb_block_claimed_bytes(int fmt, uint32_t n);   // buffer size that holds any stream of n weights in this format

// ---- block codec ----------------------------------------------------------------------------
// Encodes n weights.  idx_out must hold tfb_block_claimed_bytes(fmt, n) bytes (cb is unused: 0 bytes).
// Returns the number of payload bytes written, or -1 (also when idx_cap is too small: nothing is written past it).
long tfb_quantize_block(int fmt, const float* w, uint32_t n, uint8_t* idx_out, size_t idx_cap);
// Decodes; tolerant of short payloads (missing bits read as zero).  Unknown formats decode zeros.
void tfb_dequantize_block(int fmt, const uint8_t* idx, size_t idx_bytes, const uint8_t* cb, size_t cb_bytes,
                          uint32_t nw, float* out);

// ---- hashing --------------------------------------------------------------------------------
void tfb_sha256(const uint8_t* data, size_t n, uint8_t out32[32]);

// ---- container reader -----------------------------------------------------------------------
typedef struct tfb_reader tfb_reader;
tfb_reader* tfb_reader_open(const char* path);   // null on I/O error; check tfb_reader_valid
int tfb_reader_valid(const tfb_reader*);
void tfb_reader_close(tfb_reader*);
uint32_t tfb_reader_version(const tfb_reader*);
uint32_t tfb_reader_flags(const tfb_reader*);
uint32_t tfb_reader_config(const tfb_reader*, uint8_t* out, uint32_t cap);   // returns config size
uint32_t tfb_reader_num_tensors(const tfb_reader*);
uint32_t tfb_reader_num_blocks(const tfb_reader*);
const char* tfb_reader_tensor_name(const tfb_reader*, uint32_t i);
// number of weights of a tensor (sum of its blocks' num_weights); -1 when absent / corrupt
long long tfb_reader_tensor_numel(const tfb_reader*, const char* name);
// dequantise a whole tensor to fp32; returns elements written or -1
long long tfb_reader_read_tensor(const tfb_reader*, const char* name, float* out, long long cap);
// format byte of the first block of a tensor (-1 when absent)
int tfb_reader_tensor_format(const tfb_reader*, const char* name);

// format bytes of every block of a tensor; returns the block count (or -1), writes at most cap entries
long tfb_reader_tensor_block_formats(const tfb_reader*, const char* name, uint8_t* out, long cap);

// ---- container writer -----------------------------------------------------------------------
typedef struct tfb_writer tfb_writer;
tfb_writer* tfb_writer_open(const char* path, uint32_t version, uint32_t flags, const uint8_t* config, uint32_t config_size);
// queue a tensor: quantised per `block` weights (reference: 32768 for Q_32 saves, 256 for quantised ones)
int tfb_writer_add_tensor(tfb_writer*, const char* name, const float* data, long long numel, int fmt, uint32_t block);
// per-block formats (a planner's mix): fmts[i] encodes weights [i * block, (i + 1) * block)
int tfb_writer_add_tensor_mixed(tfb_writer*, const char* name, const float* data, long long numel, const uint8_t* fmts,
                                uint32_t nfmts, uint32_t block);
// writes header | tables | blocks in the order the reference reader expects, plus "<path>.idx"; returns 0 on success
int tfb_writer_close(tfb_writer*, int write_idx);

// ---- optimizer state (".opt") ---------------------------------------------------------------
// {i32 step, f32 lr, i32 num_params, per param: i64 n_m, m floats, i64 n_v, v floats}
int tfb_opt_write(const char* path, int step, float lr, int num_params, const long long* sizes, const float* const* m,
                  const float* const* v);
int tfb_opt_read_header(const char* path, int* step, float* lr, int* num_params);
int tfb_opt_read(const char* path, int num_params, const long long* sizes, float* const* m, float* const* v);

#ifdef __cplusplus
}
#endif
