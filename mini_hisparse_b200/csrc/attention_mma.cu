// Causal grouped-query attention over the paged KV cache on the tensor cores (bfloat16 inputs,
// float32 scores, softmax and accumulation), for prefill portions and decode tokens alike.
//
// Math as in attention_simt.cu (mini_hisparse/model.py:173-179, mini_hisparse/attention.py:26-35):
// s_t = (K[t] . q) * scale over the cached keys t <= the query's position (and inside the window,
// if there is one), w = softmax(s), o = sum_t w_t V[t]; query head h reads KV head h / groups.
// The work items are the same 8 ints {segment, first token, tokens, first head of the group,
// heads, kv_begin, kv_end, split}; split >= 0 writes an un-normalised partial.  With a counter
// array the CTA that finishes a token's last split merges all its splits (in split order, so the
// result does not depend on which CTA comes last); without one, attention_combine does it.
//
// One CTA (4 warps) serves one item and one KV head.  The query heads of a KV group are stacked
// into the row dimension of the tile, so a page of keys is read once for the whole group.
//   ROWS = 64 (long portions): each warp owns 16 query rows and walks all keys.
//   ROWS = 16 (decode tokens, tiny portions): the four warps share the 16 rows and each takes
//     16 of the 64 keys of a tile; their partial results are merged at the end.
// Keys and values arrive in tiles of 64 by cp.async (16-byte chunks gathered through the block
// table, two or three stages deep); rows are padded by 16 bytes, which keeps ldmatrix conflict-free for
// every head size that is a multiple of 16.  Products are mma.sync m16n8k16: the score tile
// feeds the value product straight from registers.
#include "attention_mma_kernel.cuh"

using namespace mhb;
using namespace mhb_amma;

MHB_EXPORT const char* mhb_last_error() { return error_buffer(); }

namespace {
template <int ROWS>
int dispatch_d(int d, const AttnArgs& a, int launch_items, cudaStream_t stream) {
    switch (d) {
        case 32: return launch<32, 32, ROWS, false>(a, launch_items, stream);
        case 64: return launch<64, 64, ROWS, false>(a, launch_items, stream);
        case 96: return launch<96, 96, ROWS, false>(a, launch_items, stream);
        case 128: return launch<128, 128, ROWS, false>(a, launch_items, stream);
    }
    return fail("attention_mma: head_dim %d has no tensor-core instance (32, 64, 96, 128)", d);
}
}  // namespace

// rows = 64 or 16: the tile height the items were planned for.
MHB_EXPORT int mhb_attention_mma(const void* q, const void* cache, void* out, float* part_acc,
                                 float* part_ml, const int* items, int num_items, int launch_items,
                                 int rows, const int* positions, const int* block_table, int width,
                                 const int* tok_part_row, const int* tok_nsplit, int* counters, int nq,
                                 int nkv, int d, int P, int num_pages, int window, float scale,
                                 cudaStream_t stream) {
    if (launch_items <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return fail("attention: %d query heads over %d KV heads", nq, nkv);
    AttnArgs a;
    fill_args(a, q, cache, out, part_acc, part_ml, items, num_items, positions, block_table, width, tok_part_row,
              tok_nsplit, counters, nq, nkv, P, num_pages, window, scale);
    if (rows == 64) return dispatch_d<64>(d, a, launch_items, stream);
    if (rows == 16) return dispatch_d<16>(d, a, launch_items, stream);
    return fail("attention_mma: tile height %d", rows);
}

MHB_EXPORT int mhb_attention_mma_supports(int d) { return d == 32 || d == 64 || d == 96 || d == 128; }
