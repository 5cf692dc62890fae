// C ABI of the host-side runtime library (no CUDA dependency).
//
//   container : memory-mapped `.mfq` reader (single file or `-NNNNN-of-NNNNN` shard set), parallel range reads
//   rows      : CPU decoders of packed weight rows (NINT v2, MXFP4, E4M3 block-scaled) -- the numerical oracle and
//               the source for embedding rows / host-resident experts
//   prefix    : content-addressed KV block store (SHA-256 chain over 256-token blocks, RAM tier + file tier)
//   planner   : tensor-parallel slice planner, MoE residency ranker, slot book, dispatch cost model
//
// Every function returns 0 (or a non-negative count / handle) on success and a negative code on failure;
// mfq_last_error() gives the message of the calling thread's last failure.
#pragma once
#include <cstddef>
#include <cstdint>

extern "C" {
const char* mfq_last_error();

// ---- container ----------------------------------------------------------------------------------------------
void* mfq_store_open(const char* path);          // a file, or any shard of a set (all shards are opened)
void mfq_store_close(void* store);
int mfq_store_version(void* store);
const char* mfq_store_arch(void* store);
int mfq_store_extra_count(void* store);
const char* mfq_store_extra_key(void* store, int i);
const char* mfq_store_extra_json(void* store, int i);
int64_t mfq_store_tensor_count(void* store);
const char* mfq_store_tensor_name(void* store, int64_t i);
const char* mfq_store_tensor_dtype(void* store, int64_t i);
int64_t mfq_store_tensor_nbytes(void* store, int64_t i);
int mfq_store_tensor_file(void* store, int64_t i);
int64_t mfq_store_find(void* store, const char* name);            // -1 if absent
const void* mfq_store_tensor_data(void* store, int64_t i);        // pointer into the mapping
// copy [offset, offset+nbytes) of a blob into dst (e.g. pinned staging) with `threads` workers; advises the kernel
// to drop the pages afterwards when drop_cache != 0
int mfq_store_read(void* store, int64_t i, int64_t offset, int64_t nbytes, void* dst, int threads, int drop_cache);

// ---- packed rows --------------------------------------------------------------------------------------------
void* mfq_nint_open(const void* blob, int64_t nbytes);            // indexes a NINT v2 payload (no copy)
void mfq_nint_close(void* h);
int64_t mfq_nint_rows(void* h);
int64_t mfq_nint_row_len(void* h);
int mfq_nint_decode(void* h, int64_t row_begin, int64_t row_end, float* out, int threads);  // out [rows, row_len]
int mfq_nint_row_bits(void* h, int64_t row, int* q_bits, int* k_bits);
// y[r] = dot(decoded row r, x) for r in [row_begin, row_end): GEMV straight from the packed payload
int mfq_nint_gemv(void* h, int64_t row_begin, int64_t row_end, const float* x, float* y, int threads);
int mfq_mxfp4_decode(const uint8_t* codes, const uint8_t* scales_e8m0, int64_t rows, int64_t cols, float* out, int threads);
int mfq_fp8_block_decode(const uint8_t* codes, const float* scales, int64_t rows, int64_t cols, int block, float* out, int threads);
// NVQ rows from the unpacked index / sign / sub-scale streams (see packed_rows.cpp); out [rows, n]
int mfq_nvq_decode(const uint16_t* indices, const uint8_t* signs, const uint8_t* sub, const float* anchors, const float* table,
                   int64_t rows, int64_t n, int gs, int vec, int entries, int index_parity, float* out, int threads);
void mfq_f32_to_bf16(const float* in, uint16_t* out, int64_t n);

// ---- prefix cache -------------------------------------------------------------------------------------------
void* mfq_prefix_open(const char* dir, int64_t ram_budget_bytes, int64_t disk_budget_bytes, int block_tokens);
void mfq_prefix_close(void* cache);
// chained keys of the full blocks of a token sequence: key[i] = SHA256(key[i-1] || tokens of block i || salt)
int mfq_prefix_keys(void* cache, const int32_t* tokens, int64_t n_tokens, const char* salt, uint8_t* keys_out /*[n_blocks,32]*/);
int mfq_prefix_put(void* cache, const uint8_t* key, const void* data, int64_t nbytes);   // async file write behind
int64_t mfq_prefix_get(void* cache, const uint8_t* key, void* dst, int64_t capacity);     // bytes, -1 if absent
int mfq_prefix_match(void* cache, const uint8_t* keys, int n_keys);                       // leading blocks present
int mfq_prefix_pin(void* cache, const uint8_t* key, int delta);
int mfq_prefix_flush(void* cache);                                                        // wait for pending writes
int mfq_prefix_stats(void* cache, int64_t* out8);  // ram_bytes, disk_bytes, ram_entries, disk_entries, hits_ram, hits_disk, misses, evictions

// ---- planners -----------------------------------------------------------------------------------------------
// contiguous slices of `total` units over `ranks` workers, proportional to weights, multiples of `granularity`
int mfq_tp_plan(int64_t total, int ranks, const double* weights, int64_t granularity, int64_t* begin_out, int64_t* end_out);
// residency ranker: given heat per expert and the resident set, propose up to max_swaps (evict, load) pairs
int mfq_moe_rank_swaps(const double* heat, const uint8_t* resident, int n_experts, int max_swaps, double hysteresis,
                       int* evict_out, int* load_out);
// per-expert execution tier for one step: 0 inactive, 1 GPU resident, 2 GPU after transfer, 3 CPU
int mfq_moe_dispatch_plan(const int* tokens_per_expert, const uint8_t* resident, int n_experts, double bytes_per_expert,
                          double h2d_gbs, double gpu_tok_us, double cpu_tok_us, int cpu_available, int* tier_out);
// ---- token constraints ----------------------------------------------------------------------------------------
// JSON grammar over a byte trie of the vocabulary (json_constraint.cpp); state = 16 opaque bytes
void* mfq_json_vocab_open(const uint8_t* bytes, const int64_t* offsets, int64_t vocab);
void mfq_json_vocab_close(void* vocab);
int64_t mfq_json_vocab_nodes(void* vocab);
void mfq_json_state_init(void* state, int need_object);
int mfq_json_state_feed(void* state, const uint8_t* bytes, int64_t n);
int mfq_json_state_complete(const void* state);
int64_t mfq_json_mask(void* vocab, const void* state, uint32_t* bits_out);

void* mfq_slotbook_open(int slots);
void mfq_slotbook_close(void* book);
int mfq_slotbook_lookup(void* book, int64_t key);                 // slot or -1; refreshes recency
int mfq_slotbook_acquire(void* book, int64_t key, int64_t* evicted_key);  // slot; evicts the LRU unpinned entry
int mfq_slotbook_pin(void* book, int64_t key, int delta);
}
