// Internal launch interfaces between the C-ABI layer (fa_api.cu) and the kernels.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace fa {

struct DecodeKernelParams {
  int* status;         // device status word
  const void* q;
  void* out;
  float* lse_out;
  const int32_t* block_table;
  const int32_t* seqlens;
  const float* q_descale;
  const float* k_descale;
  const float* v_descale;
  float* o_partial;    // [partition][b][h][sq][d] fp32
  float* lse_partial;  // [partition][b][h][sq] fp32, natural log, -inf = no keys
  int64_t q_batch_stride, q_head_stride, q_row_stride;
  int64_t o_batch_stride, o_head_stride, o_row_stride;
  int64_t bt_stride;
  int64_t qds_b, qds_h, kds_b, kds_h, vds_b, vds_h;
  int32_t b, h, h_k, group;
  int32_t page_size, box_tok;
  int32_t partition_tokens, num_partitions;
  int32_t out_dtype;
  int32_t write_final;
  float scale_log2;
  const void* s_aux;   // attention sinks (h), applied where the row is finalised (write_final only)
  int32_t s_aux_dtype;
  int32_t window_left; // the query token sees only its last window_left + 1 keys; -1 = all
  int32_t v_transposed; // tmap_v describes (page tokens, d, h_k, block) with a (64, 128, 1, 1) box
  int32_t sq;           // query tokens per sequence, the last sq positions of it; sq * group <= 16 rows of the MMA tile
  int32_t causal;       // sq > 1: token s sees the keys up to its own position
  int32_t kv_e4m3;      // the cache is e4m3 while the queries are 16-bit (launch_decode's dtype is then the query type)
  int32_t d;            // head dimension: 128, or 64 / 192 / 256 with 16-bit pools
  int32_t kv_e5m2;      // with kv_e4m3: the cache bytes are e5m2
  int32_t max_len;      // tokens the block table (and the partition grid) covers: longer cache_seqlens entries are cut
                        // to it and reported through the status word
  // Split mode with the merge inside this kernel: one int per (sequence, kv head), zero before the launch.  Every CTA
  // that wrote a partial takes a ticket; the one that takes the last ticket of its (sequence, kv head) merges that
  // pair's partials into out / lse_out (out_dtype -1: fp32) and puts the ticket back to zero.  nullptr: the partials
  // are left for the combine kernel.
  int* tickets;
  int32_t merge_lse_empty_is_neg;   // merged rows without keys: LSE -inf (partial convention) instead of +inf
  int32_t merge_sink;               // the merge adds the sink (s_aux) to the row sums
  int32_t dependent_launch;         // launch with programmatic stream serialisation (the kernel waits by itself)
  int32_t test_withhold;            // FA_B200_TEST_HOOKS builds only: CTA (0, 0, 0) announces its first tile and never loads it
};

int decode_max_pages_per_partition();
// One CTA per (token partition, kv head, sequence): partials in o_partial / lse_partial as documented above.
cudaError_t launch_decode(int dtype, const CUtensorMap& tmap_k, const CUtensorMap& tmap_v,
                          const DecodeKernelParams& p, cudaStream_t stream);

struct CombineKernelParams {
  const float* o_partial;    // [num_parts][rows][d], partitions o_part_stride floats apart
  const float* lse_partial;  // [num_parts][rows], partitions lse_part_stride floats apart
  int64_t o_part_stride, lse_part_stride;
  void* out;
  float* lse;
  const int32_t* seqlens;    // optional: row r uses ceil(seqlens[r / h] / partition_tokens) parts
  const int32_t* parts_per_row;  // optional explicit count per batch entry
  int64_t out_row_stride;    // rows are (b, h, tok): element offset = b * out_batch_stride + h * out_row_stride + tok * out_tok_stride
  int64_t out_batch_stride;
  int64_t out_tok_stride;
  int32_t sq;                // query tokens per (sequence, head); rows = b * h * sq
  int32_t num_parts, rows, h;
  int32_t d;                 // head dimension (64, 128, 192 or 256)
  int32_t partition_tokens;
  int32_t out_dtype;         // FA_B200_F16 / BF16, or -1 for fp32
  int32_t lse_empty_is_neg;  // write -inf (partial convention) instead of +inf for rows with no keys
  float out_scale;
  const void* s_aux;         // attention sinks (h): one more term of every row's sum
  int32_t s_aux_dtype;
  int32_t dependent_launch;  // launch with programmatic stream serialisation (the kernel waits by itself)
};
cudaError_t launch_combine(const CombineKernelParams& p, cudaStream_t stream);

// Exchange of the ranks' split-KV partials over peer memory, fused with their combine (fa_exchange.cu).
constexpr int kMaxExchangeRanks = 16;
struct ExchangeKernelParams {
  int* status;               // device status word
  const float* o_local;      // (rows, d) this rank's partial
  const float* lse_local;    // (rows)
  void* peers[kMaxExchangeRanks];   // every rank's exchange buffer as mapped on this GPU (peers[rank]: its own)
  size_t region_bytes;       // one half of a buffer: exchange_region_bytes(world, rows, d)
  void* out;
  float* lse;
  int64_t out_batch_stride, out_row_stride, out_tok_stride;
  int32_t world, rank, rows, h, sq, d;
  uint32_t epoch;            // > 0, one more on every call, the same on every rank
  int32_t out_dtype;         // FA_B200_F16 / BF16, or -1 for fp32
  const void* s_aux;
  int32_t s_aux_dtype;
  int32_t do_push, do_wait;  // both set in normal use; separately for single-GPU tests of the two halves
  int32_t dependent_launch;  // launch with programmatic stream serialisation (the kernel waits by itself)
};
size_t exchange_region_bytes(int world, int rows, int d);
cudaError_t launch_exchange_combine(const ExchangeKernelParams& p, cudaStream_t stream);

// Prefill (dense / varlen / block-sparse) on tcgen05.
struct PrefillKernelParams {
  int* status;         // device status word
  void* out;
  float* lse;
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  const float* q_descale;
  const float* k_descale;
  const float* v_descale;
  const int32_t* block_count;
  const int32_t* block_offset;
  const int32_t* column_count;   // sparse lists: must be zero everywhere (a non-zero entry raises a status bit)
  // paged K/V (one-tile kernel only): k/v tensor maps are (d, h_k, row in page, page); keys of sequence b are the
  // first seqused_k[b] rows of the pages block_table[b * bt_stride + 0..]
  const int32_t* block_table;
  const int32_t* seqused_k;
  int64_t bt_stride;
  int32_t paged, page_size, box_rows;
  int64_t max_keys;        // paged: keys the block table covers (0 = unknown); longer seqused_k entries are cut and reported
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t qds_b, qds_h, kds_b, kds_h, vds_b, vds_h;
  int64_t total_q;
  int32_t b, h, h_k, seqlen_q, seqlen_k;
  int32_t num_m_blocks;      // ceil(max seqlen_q / 128)
  int32_t is_causal;
  // Sliding window (bottom-right aligned like the causal mask): query row i of a sequence with sq queries and sk keys
  // sees key j iff  i + sk - sq - window_left <= j <= i + sk - sq + window_right;  -1 = unbounded on that side.
  // A causal mask is window_right = 0 (set by the host whenever is_causal is).
  int32_t window_left, window_right;
  int32_t out_dtype;
  int32_t num_q_blocks, nnz_s, block_m;  // sparse metadata geometry
  int32_t sparse;
  int32_t o_tma;             // the output tensor map is valid: full 128-row tiles are stored through it
  float scale_log2;
  const void* s_aux;         // attention sinks (h), applied in the epilogue
  int32_t s_aux_dtype;
  int* work_counter;         // persistent kernels: zeroed before the launch; CTAs claim work items past their first from it
  int32_t d;              // head dimension: 128, or 64 / 192 / 256 (16-bit types, one-tile kernel)
  int32_t d_v;            // head dimension of v and out (= d, or 128 with d = 192)
  int32_t v_transposed;   // paged V pool with the tokens contiguous: tmap_v describes (page tokens, d, h_k, block), box (64, 128, 1, 1)
  int32_t test_withhold;  // FA_B200_TEST_HOOKS builds only: CTA 0 announces the first K tile of its first item and never loads it
};
// One 128-row query tile per CTA, two CTAs per SM: block-sparse lists and odd GQA groups.
cudaError_t launch_prefill_single(int dtype, const CUtensorMap& tmap_q, const CUtensorMap& tmap_k,
                                  const CUtensorMap& tmap_v, const PrefillKernelParams& p, cudaStream_t stream);
// Persistent CTAs, one query tile per work item, double-buffered scores: dense / varlen prefill (default).
cudaError_t launch_prefill_dense(int dtype, const CUtensorMap& tmap_q, const CUtensorMap& tmap_k,
                                 const CUtensorMap& tmap_v, const PrefillKernelParams& p, cudaStream_t stream);
// Persistent CTAs, two query heads of one GQA group per work item: dense / varlen prefill with an even group.
// tmap_o: (d, h, rows, batch) map of the output with a (64 columns, 1, 128 rows, 1) box, used when p.o_tma is set.
cudaError_t launch_prefill_pair(int dtype, const CUtensorMap& tmap_q, const CUtensorMap& tmap_k,
                                const CUtensorMap& tmap_v, const CUtensorMap& tmap_o, const PrefillKernelParams& p,
                                cudaStream_t stream);


// KV-cache append + rotary embedding (one launch before the attention of a decode / chunked-prefill step).
struct KvAppendKernelParams {
  int* status;         // device status word
  const void* k_new;
  const void* v_new;
  const void* q;
  void* q_out;
  void* k_cache;
  void* v_cache;
  const int32_t* block_table;
  const int32_t* seqlens_k;
  int32_t* seqlens_out;
  const void* cos;
  const void* sin;
  int64_t kn_b, kn_r, kn_h, vn_b, vn_r, vn_h;
  int64_t q_b, q_r, q_h, qo_b, qo_r, qo_h;
  int64_t kc_blk, kc_row, kc_h, vc_blk, vc_row, vc_h;
  int64_t bt_stride;
  int32_t b, seqlen_q, seqlen_new, h, h_k;
  int32_t page_size, num_blocks, max_blocks_per_seq;
  int32_t rotary_dim, seqlen_ro, interleaved, q_per_token;
};
cudaError_t launch_kv_append(int dtype, const KvAppendKernelParams& p, cudaStream_t stream);


// Callers' glue (fa_glue.cu): padding removal and block-map conversion.
cudaError_t launch_read_stream(const void* src, int64_t bytes, uint32_t* sink, cudaStream_t stream);
cudaError_t launch_unpad_plan(const void* mask, int elem, int b, int s, int64_t row_stride, int32_t* seqlens,
                              int32_t* cu_seqlens, int64_t* indices, int32_t* stats, cudaStream_t stream);
cudaError_t launch_move_rows(const void* src, const int64_t* indices, void* dst, int64_t n_rows, int64_t row_bytes,
                             int64_t limit_rows, bool scatter, cudaStream_t stream);
cudaError_t launch_block_map(const uint8_t* map, int32_t* offset, int32_t* count, int64_t rows, int k, int scale, int fill,
                             cudaStream_t stream);

// Mean-similarity choice of key tiles (fa_block_select.cu).
struct BlockPoolParams {
  const void* x;             // (b, h, n, d) 16-bit, strides in elements, last dim contiguous
  int64_t batch_stride, head_stride, row_stride;
  int32_t b, h, n, d, dtype;
  int32_t block_rows, num_blocks;
  const float* sim_threshold;   // (h)
  void* pooled;              // (b, h, num_blocks, d), element type of x
  uint8_t* sim;              // (b, h, num_blocks)
};
struct BlockSelectParams {
  const void* pooled_q;      // (b, h, nq, d)
  const void* pooled_k;      // (b, h, nk, d)
  const uint8_t* sim_q;      // (b, h, nq)
  const uint8_t* sim_k;      // (b, h, nk)
  int32_t dtype, b, h, nq, nk, nk_pow2, d;
  int32_t block_q, block_k;  // rows per query / key block (causal mask between blocks)
  float scale;
  const float* cdf_threshold;   // (h), or
  const float* topk;            // (h): fraction of the key blocks to keep
  int32_t is_causal, attention_sink;
  uint8_t* block_map;        // (b, h, nq, nk)
};
int block_select_max_key_blocks();
cudaError_t launch_block_pool(const BlockPoolParams& p, cudaStream_t stream);
cudaError_t launch_block_select(const BlockSelectParams& p, cudaStream_t stream);

}  // namespace fa
