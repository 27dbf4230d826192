// Decode attention over the paged cache with the library's own scratch memory.
//
// This entry point has no counterpart in the reference (ZacWalk/nncpu runs on
// the CPU and sizes all of its scratch when a session is made).  It exists for
// callers of this library that cannot allocate device memory themselves:
//   * a host process that has already handed all free GPU memory to its own
//     pools, for which cudaMalloc would simply fail;
//   * a plugin, or a binding from another language, that only ever receives raw
//     device pointers and has no allocator to ask;
//   * a latency-critical loop that must stay out of the driver's allocator,
//     because an allocation may stall every stream of the device.
// Such a caller still passes its inputs and its output; only the scratch that
// the split-key kernel merges through comes from the library: a fixed
// __device__ array of nncpu_attention_decode_mma_static_max_floats() floats
// (4 MiB) that every GPU loading the library keeps until the process ends.
//
// Rules of use:
//   * The first call on each device looks the array's address up (with that
//     device current).  Make that first call before any stream capture begins.
//   * No call allocates or frees memory.
//   * All calls on a device share the array and it keeps the last call's
//     contents; no part of it needs clearing, since each call writes everything
//     it later reads.  Calls that overlap on the GPU race on it: issue them on
//     one stream, or order them yourself.
//   * Sizes that need more than the array holds are refused with a message
//     (nncpu_last_error_attention_mma) and a non-zero return value; nothing is
//     launched.  The need is n_tok * n_kv * n_splits * (n_heads / n_kv) * (hd + 2)
//     floats for n_splits > 1 and nothing for n_splits == 1.
//
// Arguments are those of nncpu_attention_decode_mma without its scratch pair:
// q, out: bfloat16 [n_tok, n_heads * hd]; k_pages, v_pages: bfloat16
// [pages, n_kv, 64, hd]; block_table: int32 [sequences, bt_stride] page ids;
// tok_seq[t]: the sequence of token t (negative: padding, output zeros);
// tok_pos[t]: its position, whose keys 0..tok_pos[t] (or the last `window`)
// are attended; hd 64 or 128; at most 16 query heads per key/value head.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

long nncpu_attention_decode_mma_static_max_floats(void);

int nncpu_attention_decode_mma_static(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                      int bt_stride, const int* tok_seq, const int* tok_pos, void* out, int n_tok,
                                      int n_heads, int n_kv, int hd, float scale, int window, int n_splits,
                                      void* stream);

#ifdef __cplusplus
}
#endif
