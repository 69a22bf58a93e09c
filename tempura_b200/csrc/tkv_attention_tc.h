// Interface between the decode-attention entry point (tkv_attention.cu) and its tcgen05 kernel (tkv_attention_tc.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tkv_tc {

// partial results one token range writes: one per softmax group of the kernel
constexpr uint32_t PARTS_PER_RANGE = 2;

struct Args {
    const float* k_scales;        // [total_blocks][8] of this layer, or null
    const float* v_scales;
    const float* q;               // [n_seqs][n_q_heads][128]
    const uint32_t* tables;       // [n_seqs][table_stride]
    const uint32_t* kv_lens;
    float* partial;               // [n_seqs][8][PARTS_PER_RANGE * n_splits][group][128 + 2]: running maximum, row sum, 128 numerators;
                                  // the kernel's softmax groups take the blocks of a range in turn and each writes its own part
    uint32_t n_seqs, n_q_heads, table_stride, n_splits, split_tokens, max_kv_len, total_blocks;
    float q_scale;                // softmax scale * log2(e)
    uint32_t* status;             // optional device word: first failure wins
};

// 8 kv heads of 128 dims in 16-token blocks (one block = one 128-row operand tile), 4 query heads per kv head
bool eligible(uint32_t n_kv_heads, uint32_t group, bool has_scales, uint32_t total_blocks);
// launches on the current device; layer tensors as raw device addresses
cudaError_t launch(bool fp8, uint32_t group, uint64_t k_layer, uint64_t v_layer, const Args& a, cudaStream_t st);

// operand plumbing of the tcgen05 path (tensor-map copy, swizzle, descriptors, tensor-memory reads) on exact small cases:
// out[0..3] = mismatches of {E4M3 K-major, E4M3 x E5M2 MN-major, F16 K-major, F16 MN-major}
cudaError_t selfcheck(uint64_t out[4]);

// ---- prefill side: causal attention of a chunk of new tokens of one sequence (tkv_prefill_tc.cu) ----
struct PrefillArgs {
    const float* k_scales;        // [total_blocks][8] of this layer, or null
    const float* v_scales;
    const float* q;               // [n_tokens][n_q_heads][128]
    float* out;                   // same shape
    const uint32_t* table;        // the sequence's block ids, at least ceil((start_pos + n_tokens) / 16) of them
    uint32_t n_tokens, start_pos, n_q_heads, total_blocks;
    float q_scale;                // softmax scale * log2(e)
    uint32_t* status;             // optional device word: first failure wins
    uint32_t single_tile;         // 1 = one query tile per CTA, 2 = two, 0 = the library's choice
};
bool prefill_eligible(uint32_t n_kv_heads, uint32_t n_q_heads, uint32_t head_dim, uint32_t block_size, uint32_t total_blocks);
cudaError_t launch_prefill(bool fp8, uint64_t k_layer, uint64_t v_layer, const PrefillArgs& a, cudaStream_t st);

}  // namespace tkv_tc
