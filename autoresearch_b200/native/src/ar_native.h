// C ABI of the host-side native library (data plane, RNG, checkpoint I/O).
//
// The reference implements these pieces in Rust inside its single binary
// (brain/src/train.rs:247-622 data loaders, :2424-2483 RNG, brain/src/feeder/*.rs,
// safetensors crate).  Here they are C++17 behind a flat C interface that Python binds
// with ctypes and that the stand-alone `feeder` binary links directly.
#pragma once
#include <cstddef>
#include <cstdint>

extern "C" {

// ---- RNG / initialisation -----------------------------------------------------------
// xorshift64 stream shared across calls through *state (seed 42 in the reference).
void ar_uniform_bf16(uint64_t* state, int64_t n, double bound, uint16_t* out);
void ar_uniform_f32(uint64_t* state, int64_t n, double bound, float* out);
void ar_randn_f32(uint64_t* state, int64_t n, float scale, float* out);
void ar_randn_bf16(uint64_t* state, int64_t n, float scale, uint16_t* out);
void ar_shuffle_order(int64_t* order, int64_t n, uint64_t seed);

// ---- synthetic token streams --------------------------------------------------------
// LCG stream of the reference (tokens in [1, vocab-1]); *state carries over.
void ar_lcg_tokens(uint64_t* state, int64_t n, uint32_t vocab, int32_t* out);
// Zipf(s) over ids [0, vocab) from a seeded splitmix64 stream; cdf is built once.
void* ar_zipf_create(uint32_t vocab, double s, uint64_t seed);
void ar_zipf_fill(void* h, int64_t n, int32_t* out);
void ar_zipf_seek(void* h, uint64_t seed, uint64_t draws);
void ar_zipf_destroy(void* h);

// ---- TKNS shards ----------------------------------------------------------------------
// returns 0 on success; negative error codes: -1 io, -2 too small, -3 magic, -4 version,
// -5 truncated
int ar_shard_open(const char* path, void** handle, uint32_t* vocab, uint32_t* seq_len,
                  uint32_t* num_rows);
const uint16_t* ar_shard_row(void* handle, uint32_t idx);
void ar_shard_close(void* handle);
int ar_shard_write(const char* path, uint32_t vocab, uint32_t seq_len, uint32_t num_rows,
                   const uint16_t* rows);

// ---- row stream (reader thread + bounded queue over a file descriptor) ---------------
// Reads rows of row_len little-endian u16 from fd on a background thread into a ring of
// `depth` batches of `batch_rows` rows.  ar_rowstream_next blocks until a batch is ready
// and writes ids/targets (int32, [batch_rows, row_len-1]) into caller memory (which may
// be pinned).  Returns 1 on success, 0 on clean end of stream, -1 if the stream ended in
// the middle of a row or the reader failed, -2 on timeout.
void* ar_rowstream_open(int fd, int32_t row_len, int32_t batch_rows, int32_t depth);
int ar_rowstream_next(void* h, int32_t* ids, int32_t* targets, int32_t timeout_ms);
int64_t ar_rowstream_rows_read(void* h);
void ar_rowstream_close(void* h);

// ---- best-fit packer --------------------------------------------------------------------
void* ar_packer_create(int32_t row_capacity, int32_t buffer_docs);
void ar_packer_add_doc(void* h, const int32_t* tokens, int32_t n);
int32_t ar_packer_buffered(void* h);
// Emits one row (row_capacity u16).  `exhausted` != 0 tells the packer that no more
// documents will arrive, which allows zero padding.  Returns 1 if a row was produced, 0
// if more documents are needed (or nothing is left).
int ar_packer_next_row(void* h, int exhausted, uint16_t* out_row);
void ar_packer_destroy(void* h);

// ---- safetensors ---------------------------------------------------------------------------
// Writer: entries must be added, then finish() writes header + data (names sorted).
void* ar_st_writer_create(void);
void ar_st_writer_add(void* w, const char* name, const char* dtype, const int64_t* shape,
                      int32_t ndim, const void* data, int64_t nbytes);
int ar_st_writer_finish(void* w, const char* path);  // 0 ok; frees the writer
// Reader: mmap + header index.
void* ar_st_open(const char* path, char* err, int32_t errlen);
int32_t ar_st_count(void* r);
const char* ar_st_name(void* r, int32_t i);
const char* ar_st_dtype(void* r, int32_t i);
int32_t ar_st_ndim(void* r, int32_t i);
int64_t ar_st_dim(void* r, int32_t i, int32_t d);
const void* ar_st_data(void* r, int32_t i, int64_t* nbytes);
void ar_st_close(void* r);

// ---- BPE vocabulary training ---------------------------------------------------------------
// words: concatenated bytes, word w = bytes[offsets[w] .. offsets[w+1]) seen counts[w] times.  Writes up to
// vocab_size-256 merges as (left id, right id) pairs (merge i creates id 256+i) and returns their number.
int32_t ar_bpe_train(const uint8_t* bytes, const int64_t* offsets, const int64_t* counts, int64_t n_words,
                     int32_t vocab_size, int32_t* merges_out);

// ---- BPE tokenizer -----------------------------------------------------------------------
void* ar_tok_load_json(const char* path, char* err, int32_t errlen);
void* ar_tok_load_tiktoken(const char* tiktoken_path, const char* config_path, char* err,
                           int32_t errlen);
int32_t ar_tok_vocab(void* t);
int32_t ar_tok_bos(void* t);
// Encodes UTF-8 text; returns number of tokens (call with out=NULL to size).
int64_t ar_tok_encode(void* t, const char* text, int64_t len, int add_bos, int32_t* out,
                      int64_t cap);
// Splits only (pre-tokenisation); writes piece end offsets; returns number of pieces.
int64_t ar_tok_split(void* t, const char* text, int64_t len, int64_t* ends, int64_t cap);
int64_t ar_tok_decode(void* t, const int32_t* ids, int64_t n, char* out, int64_t cap);
void ar_tok_destroy(void* t);

}  // extern "C"
