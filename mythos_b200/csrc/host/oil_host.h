// C ABI of the host runtime library (liboil_host.so): the .oil container (mmap reader with an
// O(1) block index, streaming writer, dequantisation of all six block formats), SHA-256, the
// .oilidx sidecar check, the byte-level BPE tokenizer, the reference-compatible RNG, the KV
// page allocator and the prefetching token-window loader. Python reaches it through ctypes (mythos_b200/oil/native_io.py); C and C++
// programs include this header. Functions return 0 / a handle on success and a negative code /
// null on failure; oil_last_error() describes the last failure of the calling thread.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* oil_last_error(void);

// ---- SHA-256
void oil_sha256(const uint8_t* data, size_t n, uint8_t out[32]);
int oil_sha256_file(const char* path, uint8_t out[32]);

// ---- container reader
typedef struct OilFile OilFile;
OilFile* oil_open(const char* path);
void oil_close(OilFile* f);
uint32_t oil_version(const OilFile* f);
uint32_t oil_config_size(const OilFile* f);
const uint8_t* oil_config(const OilFile* f);
uint32_t oil_num_tensors(const OilFile* f);
uint32_t oil_num_blocks(const OilFile* f);
const char* oil_tensor_name(const OilFile* f, uint32_t i);
int64_t oil_tensor_numel(const OilFile* f, const char* name);
// Dequantises the whole tensor into out[0..numel). Returns the element count or a negative code.
int64_t oil_read_tensor_f32(const OilFile* f, const char* name, float* out, int64_t capacity);
int oil_block_info(const OilFile* f, uint32_t block, uint8_t* format, uint32_t* num_weights, uint64_t* offset,
                   uint32_t* cb_bytes, uint32_t* idx_bytes);
int oil_tensor_sha256(const OilFile* f, const char* name, uint8_t out[32]);

// ---- container writer (header -> format table -> tensor table -> blocks, as the reference)
typedef struct OilWriter OilWriter;
OilWriter* oil_writer_create(const char* path, const uint8_t* config, uint32_t config_size, uint32_t version,
                             uint32_t flags);
int oil_writer_add_tensor(OilWriter* w, const char* name);  // following blocks belong to this tensor
int oil_writer_add_block(OilWriter* w, uint8_t format, uint32_t num_weights, const uint8_t* cb, uint32_t cb_bytes,
                         const uint8_t* idx, uint32_t idx_bytes);
int oil_writer_finish(OilWriter* w);  // writes the file atomically and frees the writer

// ---- sidecar: returns the number of tensors, or -(index+1) of the first corrupt / truncated record
int oil_idx_check(const char* path, char* bad_name, size_t bad_name_cap);

// ---- BPE tokenizer (.vocab layout of the reference)
typedef struct OilBpe OilBpe;
OilBpe* oil_bpe_train(const uint8_t* text, size_t n, int vocab_size);
OilBpe* oil_bpe_load(const char* path);
int oil_bpe_save(const OilBpe* t, const char* path);
void oil_bpe_free(OilBpe* t);
int oil_bpe_vocab_size(const OilBpe* t);
int64_t oil_bpe_encode(const OilBpe* t, const uint8_t* text, size_t n, int32_t* out, int64_t capacity);
int64_t oil_bpe_decode(const OilBpe* t, const int32_t* ids, int64_t n, uint8_t* out, int64_t capacity);

// ---- RNG: splitmix64-seeded xoroshiro128+ with 53-bit uniforms and Box-Muller normals
typedef struct OilRng OilRng;
OilRng* oil_rng_create(uint64_t seed);
void oil_rng_free(OilRng* r);
uint64_t oil_rng_next(OilRng* r);
double oil_rng_uniform(OilRng* r);
double oil_rng_normal(OilRng* r);
void oil_rng_fill_uniform(OilRng* r, float* out, int64_t n, float lo, float hi);

// ---- KV page allocator (free list + reference counts)
typedef struct OilPages OilPages;
OilPages* oil_pages_create(int32_t num_pages);
void oil_pages_free(OilPages* p);
int32_t oil_pages_alloc(OilPages* p);              // -1 when exhausted
void oil_pages_retain(OilPages* p, int32_t page);
void oil_pages_release(OilPages* p, int32_t page);
int32_t oil_pages_used(const OilPages* p);

// ---- token-window loader: windows of seq + 1 tokens, optional per-epoch window shuffle, batches
// prepared by a worker thread into a ring of `prefetch` slots (loader.cpp)
typedef struct OilLoader OilLoader;
OilLoader* oil_loader_create(const int32_t* tokens, int64_t n_tokens, int batch, int seq, int shuffle, uint64_t seed,
                             int prefetch);
int64_t oil_loader_num_batches(const OilLoader* L);
void oil_loader_reset(OilLoader* L, int epoch);
int oil_loader_next(OilLoader* L, int32_t* ids_out, int32_t* targets_out);   // 1, or 0 at the end of the epoch
void oil_loader_free(OilLoader* L);

#ifdef __cplusplus
}
#endif
