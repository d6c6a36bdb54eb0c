// Argument blocks of the attention kernels.
#pragma once
#include "common.cuh"

#define SPITE_WINDOW_FULL 0      // keys 0..pos
#define SPITE_WINDOW_CHUNK 1     // keys of the query's chunk: floor(pos/size)*size .. pos
#define SPITE_WINDOW_SLIDING 2   // the last `size` keys: max(0, pos-size+1) .. pos

// The tokens of one step, flattened.  Token t belongs to segment seg_of_token[t]
// (one segment per request in the step) and sits at absolute position positions[t].
// block_table[seg * table_width + p / page_size] is the page that holds position p.
struct StepTokens {
    const int* positions;
    const int* seg_of_token;
    const int* block_table;
    int table_width;
    int n_tokens;
};

// One cache: keys at kv, values at kv + v_offset (elements); a page holds, for every
// kv head, page_size rows of head_dim elements: [pages][kv heads][page_size][head_dim].
struct PagedCache {
    void* kv;
    long long v_offset;
    int n_pages;
    int page_size;
    int num_kv_heads;
    int head_dim;
};

#define SPITE_PAIR_NEIGHBOURS 0   // pair i of a head is elements (2i, 2i+1)
#define SPITE_PAIR_HALVES 1       // pair i is elements (i, i + rotary_dim/2)

struct QkPrepareParams {
    const void* qkv;            // [tokens, (nq + 2 nkv) * head_dim]: q heads, k heads, v heads
    void* q_out;                // [tokens, nq * head_dim]
    const float* inv_freq;      // [rotary_dim / 2] rotation frequencies, or null: no rotation
    const float* q_gain;        // [head_dim] gain of the norm of q heads, or null (weightless)
    const float* k_gain;        // [head_dim] the same for k heads
    float qk_norm_eps;          // > 0: RMS norm of every q and k head
    int norm_before_rotation;   // the norm runs before the rotation instead of after it
    int pairing;                // SPITE_PAIR_*
    int rotary_dim;             // the first rotary_dim elements of a head rotate (even, <= head_dim)
    int temperature_floor;      // > 0: q *= ln(floor((pos+1)/floor) + 1) * temperature_scale + 1
    float temperature_scale;
    int num_heads;
    int write_cache;            // append k and v to the cache
};

struct AttentionParams {
    const void* q;              // [tokens, nq * head_dim]
    void* out;                  // [tokens, nq * head_dim]
    int num_heads;
    int window_kind;
    int window_size;
    float softmax_scale;
};

// What the tensor-core attention kernels need beyond the above.  Two kernels share a step:
// segments of few tokens (decode) go to the one that splits the keys among blocks, segments
// of many tokens (prompt portions) to the one that gives every warp its own rows; each kernel
// serves the segments whose token count lies in [seg_min_tokens, seg_max_tokens].
struct AttnMmaExtra {
    const int* cu_seqlens;       // [segments + 1]
    float* o_part;               // [tokens, heads, splits, head_dim]   (splits > 1)
    float* ml_part;              // [tokens, heads, splits, 2]          running maximum, sum
    int n_segments;
    int tokens_per_block;        // tokens whose (token, head) rows fill one block
    int n_splits;
    int seg_min_tokens;
    int seg_max_tokens;
};

// The same for the decode kernel whose last-arriving block merges the key splits itself.
struct AttnDecodeExtra {
    const int* cu_seqlens;       // [segments + 1]
    float* partial;              // [blocks, kv heads, splits, 16, head_dim + 4]   (splits > 1)
    int* tickets;                // [blocks, kv heads], zero between launches      (splits > 1)
    int n_segments;
    int tokens_per_block;
    int n_splits;
    int seg_min_tokens;
    int seg_max_tokens;
    int cache_settled;           // the cache rows of positions before each request's first token of this step were
                                 // written at least two launches ago on this stream: they may be read before the wait
};

__device__ __forceinline__ int window_lowest(int kind, int size, int pos) {
    if (kind == SPITE_WINDOW_CHUNK) return (pos / size) * size;
    if (kind == SPITE_WINDOW_SLIDING) return max(0, pos - size + 1);
    return 0;
}
