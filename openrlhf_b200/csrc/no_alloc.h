// Allocation-free entry point of the kernel library. It has no counterpart in the reference (OpenRLHF ships no
// native code); it exists for callers of this library that are not allowed to allocate device memory.
//
// Who those callers are: code that runs while the CUDA allocator must not be touched, for example a host thread
// that drives decode steps while another thread of the process owns the caching allocator, code running inside a
// memory-pool "sleep" phase where the pool has been released to another engine, or an embedding runtime (C, Rust,
// a plugin ABI) that only holds device pointers handed to it and has no allocator at all. For them the split-KV
// decode attention, whose partial results normally go to a caller-provided workspace, is offered in a variant whose
// workspace is a fixed array inside the library's own device image.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch can hold: B * Hq * splits must not exceed this many partial rows.
#define B200_NOALLOC_MAX_PARTIAL_ROWS 8192

// Paged-KV decode attention with split-KV, same arguments and results as b200_attn_decode, minus the two workspace
// pointers. The partial outputs (fp32 [rows, 128]) and their softmax statistics ([rows, 2]) live in a file-scope
// device array of B200_NOALLOC_MAX_PARTIAL_ROWS rows (about 4.1 MB), which every GPU that loads the library holds
// until the process exits.
//
//  * Calls no cudaMalloc / cudaFree and no allocating library routine.
//  * The first call on each device resolves the array's device address (cudaGetSymbolAddress with that device
//    current) and raises the kernel's shared-memory limit; make that first call before starting any stream capture.
//  * All calls on a device share the one array. Every partial row a call reads is written by that same call first,
//    so nothing needs clearing between calls; but two calls whose kernels overlap on the GPU (different streams,
//    or graphs replayed concurrently) race on it. Serialise them on one stream.
//  * Returns 0 on a successful launch, -20 if B * Hq * splits exceeds the maximum, -21 if the symbol address cannot
//    be resolved, and the codes of b200_attn_decode otherwise.
int b200_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                             const int* seq_lens, void* out, int B, int Hq, int Hkv, int num_pages, int max_pages,
                             int splits, float scale, int* status, void* stream);

#ifdef __cplusplus
}
#endif
