/* sp_flash_decode_static: decode attention for callers that may not allocate device memory.
 *
 * This entry point has no counterpart in Erik-cpu-create/spissa (a CPU runtime without device
 * memory); it exists for programs that embed this library next to their own memory management.
 *
 * Who needs it. The regular entry point, sp_flash_decode, wants a scratch buffer and a block of
 * arrival counters from its caller, and callers normally get those from an allocator. Some cannot:
 * a server that handed every free byte of the GPU to its own pool when it started and has no
 * allocator call left to make; a plug-in whose host forbids allocation after start-up so that its
 * memory use stays what was agreed; a latency path that must not take the allocator's locks or
 * trigger its synchronisation. For them the scratch lives inside the library: a file-scope device
 * array that every GPU which loads the library holds from load to exit.
 *
 * Limits. The array holds SP_FLASH_DECODE_STATIC_MAX_FLOATS floats (4 MiB) for the per-chunk partial
 * results, n_seqs * num_heads * n_chunks * (head_dim + 2) of which a call uses, and
 * SP_FLASH_DECODE_STATIC_MAX_COUNTERS integers, n_seqs * num_kv_heads of which a call uses. A call
 * that needs more is refused with a message (return code 1, text from sp_attention_last_error); it
 * never falls back to allocating.
 *
 * Set-up. The first call on a device looks up the device addresses of the arrays with
 * cudaGetSymbolAddress while that device is current and remembers them for that device. The first
 * call on a device of each kernel variant (one per head size, 64 or 128, and per number of query
 * heads per kv head, up to 8 or up to 16) also asks that device for the kernel's shared memory and
 * loads the kernel. Make these first calls, one per shape you will use on each device, outside any
 * stream capture. What is remembered is written without a lock: two host threads that make a first
 * call at the same moment both do the set-up and store the same values, which is harmless, but let
 * one thread finish its first call where you can. No call allocates or frees anything, through CUDA
 * or any other library.
 *
 * Sharing. All calls on a device use the same array. A call clears the counters it is going to use
 * (cudaMemsetAsync on its stream) and overwrites the partial results it needs, so what an earlier
 * call left behind does no harm. Two calls whose kernels overlap on the GPU (different streams
 * without an ordering between them) race on the array; order them.
 *
 * Arguments are those of sp_flash_decode without scratch and counters: q [n_seqs, num_heads*head_dim]
 * bfloat16, out the same shape in bfloat16 (out_dt 1) or float32 (out_dt 0), paged key and value
 * pools, seq_len (lengths including the query token), seq_row, the page table, and the split of the
 * keys into n_chunks chunks of chunk_tiles pages.
 */
#pragma once
#include <cuda_runtime.h>

#define SP_FLASH_DECODE_STATIC_MAX_FLOATS (1 << 20)
#define SP_FLASH_DECODE_STATIC_MAX_COUNTERS 4096

#ifdef __cplusplus
extern "C"
#endif
int sp_flash_decode_static(const void* q, void* out, int out_dt, const void* kpool, const void* vpool,
                           const int* seq_len, const int* seq_row, const int* page_table, int max_pages,
                           int page_size, int n_seqs, int nh, int nkv, int hd, int window, float scale,
                           int chunk_tiles, int n_chunks, cudaStream_t stream);
