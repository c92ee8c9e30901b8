/* C ABI of libuq_b200.so: paged UltraQuant FP4 verify/decode attention and KV append for NVIDIA B200
 * (sm_100a).  Plain pointers and sizes only; every function returns a cudaError_t value as int
 * (0 = success, 1 = cudaErrorInvalidValue = "this shape is not served", nothing was enqueued).
 * All launches are asynchronous on `stream` (a cudaStream_t passed as void*), allocate nothing and
 * never read device memory on the host.  Pointers are caller-owned device memory.
 * Alignment: q and kc 16 bytes, mo 8 bytes, ml / out / block_table / seq_lens 4 bytes; a pointer that breaks this is
 * refused with cudaErrorInvalidValue before anything is enqueued.  (vc, ks, vs: any alignment; 16-byte aligned ones - 32
 * for kc at head_dim 128 - let the call run on the tcgen05 kernel instead of the CUDA-core one.)
 * First call: the first uqb_decode_* / uqb_tree_* / uqb_merge_wait_* call on each device loads the library's device
 * module (which carries the 24 MiB array of uqb_decode_launch_static whether or not that entry is ever used), looks up
 * per-device addresses and sets kernel attributes; make it outside any stream capture.  Device indices 0..63.
 *
 * Each function names the reference interface it stands in for (reference file:line), or says that
 * the reference has no counterpart. */
#ifndef UQ_B200_H_
#define UQ_B200_H_
#include <stddef.h>
#include <stdint.h>

#include "uq_params.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- the reference's surface, C linkage ------------------------------------------------------ */

/* uq_block_m (reference cuda/uq_decode.h:33, cuda/uq_decode.cu:398) */
int uqb_block_m(int K, int HQ, int HKV);
/* uq_mo_elems / uq_ml_elems / uq_workspace_bytes (reference cuda/uq_decode.h:34-35,41) */
size_t uqb_mo_elems(const UQParams* p);
size_t uqb_ml_elems(const UQParams* p);
size_t uqb_workspace_bytes(const UQParams* p);
/* uq_decode_launch (reference cuda/uq_decode.h:39, cuda/uq_decode.cu:602-626) */
int uqb_decode_launch(const UQParams* p, int nwarps, int stages, void* stream);
/* uq_decode_launch_ws (reference cuda/uq_decode.h:42, cuda/uq_decode.cu:629-632): workspace = mo then ml */
int uqb_decode_launch_ws(const UQParams* p, void* workspace, int nwarps, int stages, void* stream);
/* uq_has_sm90 (reference cuda/uq_decode.h:43): always 0 here */
int uqb_has_sm90(void);

/* ---- KV append-quantize ---------------------------------------------------------------------- */

/* Quantize T new tokens and scatter them into the paged cache; bit-exact with the reference encoder.
 * Stands in for uqmt.vllm_adapter.append_kv (reference uqmt/vllm_adapter.py:48-59) and for
 * uqmt.quant.quantize_on_write, rule "ceil" (reference uqmt/quant.py:157-206); the reference has no
 * native entry point for it.
 *   key, value   [T, HKV, D] contiguous; dtype 0 = fp32, 1 = bf16, 2 = fp16.  value may be NULL with
 *                vc/vs NULL to write only one stream (the quantize_on_write form).
 *   slots        int64 [T]: physical_page * PAGE + offset; a negative slot is skipped (padding).
 * D in {64,128,256}; PAGE any positive value. */
int uqb_append_launch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const void* key, const void* value,
                      const int64_t* slots, int T, int HKV, int D, int PAGE, int dtype, void* stream);

/* The same with the options of the reference's configurable quantiser (reference uqmt/quant.py):
 *   flags & 1   the KEY rows are rotated by the orthonormal Walsh-Hadamard transform over head_dim before they are
 *               encoded (fwht, uqmt/quant.py:84-98: the transform in fp32, its result rounded to the input's type);
 *               values are never rotated.  The queries of such a cache go through uqb_fwht_launch first.
 *   flags & 2   scale rule 'paper': E = round(log2(c * amax)), half to even, values clipped at +-6
 *               (scale_exponent, uqmt/quant.py:52-60; quantize_on_write(rule="paper", c), :197-206); c > 0.
 *   flags & 4 / flags & 8   take the bulk kernel / the kernel with one warp per row, whatever the size of the call (both
 *               write the same bytes; without either bit a call of 4096 or more rows x streams whose key / value pointers
 *               are 16-byte aligned goes to the bulk kernel, which runs a prompt's worth of rows at memory bandwidth;
 *               flags & 4 on a call the bulk kernel does not serve is cudaErrorInvalidValue).
 * flags = 0 is uqb_append_launch.  Bit-exact with quantize(fwht(key), rule, c) of the reference's CPU functions. */
int uqb_append_ex_launch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const void* key, const void* value,
                         const int64_t* slots, int T, int HKV, int D, int PAGE, int dtype, int flags, float c, void* stream);

/* The append for an NVFP4 cache (UQParams.fmt = 1): codes as above, one e4m3fn scale byte per 16 channels (ks / vs
 * [pages, HKV, PAGE, D/16]) for the per-tensor fp32 scales k_ts / v_ts (> 0), which the caller keeps and passes to the
 * decode launch.  Bit-exact with the reference's quantiser quantize_nvfp4(x, tensor_scale) (uqmt/quant.py:125-136; paged
 * cache uqmt/nvfp4.py:229-254); the reference has no kernel for it.  key and value both required. */
int uqb_append_nvfp4_launch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const void* key, const void* value,
                            const int64_t* slots, int T, int HKV, int D, int PAGE, int dtype, float k_ts, float v_ts, void* stream);
/* The same with a choice of kernel: flags 0 = by the size of the call (uqb_append_nvfp4_launch), 4 = the bulk kernel,
 * 8 = the kernel with one warp per row; same bytes (see uqb_append_ex_launch). */
int uqb_append_nvfp4_ex_launch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const void* key, const void* value,
                               const int64_t* slots, int T, int HKV, int D, int PAGE, int dtype, float k_ts, float v_ts, int flags,
                               void* stream);

/* Orthonormal Walsh-Hadamard transform along the last axis of x [rows, D] (D in {64,128,256}; dtype as above),
 * out may be x: the reference's fwht (uqmt/quant.py:84-98, rotate_kq :105-107) for the queries. */
int uqb_fwht_launch(const void* x, void* out, long long rows, int D, int dtype, void* stream);

/* ---- the upstream engines' slot layout ------------------------------------------------------------ */

/* Byte permute between this library's four cache arrays and the upstream engines' single array of per-token slots
 * [pages, PAGE, HKV, slot_bytes], slot = K codes (D/2) | K scale bytes (D/32) | V codes | V scale bytes | padding: the
 * converter of the reference's compatibility notes (reference cuda/UPSTREAM_COMPAT.md:81-88, torch permute / cat there).
 * slot_bytes >= D + D/16.  flags of the outbound direction: 1 = a minus-zero code nibble (0x8) is written as 0x0
 * (canon_negzero, reference cuda/compat/paper_rule_cpu_check.py:14-18), 2 = a 32-channel group whose codes are all zero
 * gets the scale byte 0, upstream's mark for an all-zero group (reference cuda/UPSTREAM_COMPAT.md:93-95); with both, a
 * cache written by uqb_append_ex_launch with the 'paper' rule holds the upstream encoder's bytes.  The inbound direction
 * is the permute alone (both layouts decode as code * 2^(byte - 127)).  kc / vc 16-byte aligned. */
int uqb_cache_to_upstream_launch(const uint8_t* kc, const uint8_t* ks, const uint8_t* vc, const uint8_t* vs, uint8_t* slots_out,
                                 long long pages, int HKV, int PAGE, int D, int slot_bytes, int flags, void* stream);
int uqb_cache_from_upstream_launch(const uint8_t* slots_in, uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs,
                                   long long pages, int HKV, int PAGE, int D, int slot_bytes, void* stream);

/* ---- context-split partials and their merge (no counterpart in the reference) ---------------- */

/* Attention of all queries over ONE SHARD of each sequence's context.  The cache and block_table in
 * `p` hold only this shard's pages; shard-local key t of sequence b is global position
 * pos_offset[b] + t and the shard holds n_local = clamp(seq_len - pos_offset, 0, max_pages*PAGE)
 * keys.  seq_lens stay global.  Writes, per query row, the normalised partial output
 * o_part fp32 [B,K,Hq,D] and lse2_part fp32 [B,K,Hq] = log2 of the sum of 2^(score*log2 e) over the
 * shard (-inf and zeros when the row sees no key of this shard).  p->out is not used.
 * pos_offset == NULL means offset 0 (the shard is the whole context). */
int uqb_decode_partial_launch(const UQParams* p, const int32_t* pos_offset, float* o_part, float* lse2_part,
                              void* stream);
/* Tree-masked verify (reference uqmt/tree.py:130-166 uq_tree_decode, oracle tree_reference :169-201; Triton only in the
 * reference, no C++ entry point).  The K draft tokens of a sequence sit at its last K positions; query j sees the whole
 * committed prefix and draft token t iff bit t of tree_mask[b*K + j] is set.  tree_mask: device int32 [B,K], K <= 16;
 * NULL = the chain mask, i.e. uqb_decode_launch.  Everything else as uqb_decode_launch. */
int uqb_tree_decode_launch(const UQParams* p, const int32_t* tree_mask, void* stream);
/* Log-sum-exp merge of R shards' partials: o_parts fp32 [R,rows,D], lse2_parts fp32 [R,rows]
 * -> out bf16 [rows,D]  (same arithmetic as the reference's in-GPU combine, cuda/uq_decode.cu:353-388). */
int uqb_merge_launch(const float* o_parts, const float* lse2_parts, int R, size_t rows, int D, void* out_bf16,
                     void* stream);
/* The same merge when every shard's partials are one packed buffer, o [rows,D] followed by lse2 [rows] (what one
 * all-gather of the ranks' buffers gives): packed fp32 [R][rows*D + rows].  No counterpart in the reference. */
int uqb_merge_packed_launch(const float* packed, int R, size_t rows, int D, void* out_bf16, void* stream);

/* ---- context split over peer memory: the partials cross NVLink by plain stores, no collective call (no counterpart
 *      in the reference, which has no multi-GPU code) ------------------------------------------------------------------
 * Every rank owns one exchange buffer of uqb_peer_bytes(world, rows, D) bytes (rows = B*K*Hq of the largest call it will
 * serve), allocated by uqb_peer_alloc, which also returns a 64-byte handle; the other ranks (one process per GPU of one
 * box) open the handle with uqb_peer_open and get a pointer to that buffer that their kernels can store through.  These
 * four calls allocate / map memory: they belong to set-up, never to the serving loop.
 * A call then is two launches per rank, both asynchronous and allocation-free:
 *   uqb_decode_partial_push_launch  attention over this rank's context shard (as uqb_decode_partial_launch); the combine
 *                                   kernel stores the packed partial (o fp32 [rows,D], then lse2 [rows]) into this rank's
 *                                   slot of EVERY rank's buffer (bases[r], r = 0..world-1, bases[rank] the local one) and,
 *                                   when its last block is done, sets this rank's flag there to `seq`;
 *   uqb_merge_wait_launch           waits until all `world` flags of the local buffer equal `seq`, then merges the slots
 *                                   to bf16 [rows,D] (the arithmetic of uqb_merge_packed_launch).
 * seq is the caller's call counter: it starts at 1, grows by one per call and is the same on every rank; slots and flags
 * are double buffered by its parity, so a rank may run one call ahead of the slowest.  The wait is bounded: after wait_ns
 * nanoseconds (0 = one second) without a rank's flag the kernel writes nothing, records code 3 with that rank and seq in
 * the status record (uqb_last_status) and returns - the output of that call is then undefined and the caller decides
 * (a rank that has left: stop using the group).  p->out, p->mo / p->ml as for uqb_decode_partial_launch (scratch needed,
 * out unused).  world <= 8.  All pointers in `bases` must be device-accessible from this rank. */
size_t uqb_peer_bytes(int world, size_t rows, int D);
int uqb_peer_alloc(size_t bytes, void** ptr, unsigned char handle64[64]);
int uqb_peer_open(const unsigned char handle64[64], void** ptr);
int uqb_peer_close(void* ptr);
int uqb_peer_free(void* ptr);
int uqb_decode_partial_push_launch(const UQParams* p, const int32_t* pos_offset, void* const* bases, int world, int rank,
                                   unsigned int seq, void* stream);
int uqb_merge_wait_launch(const void* own_base, int world, unsigned int seq, size_t rows, int D, void* out_bf16,
                          unsigned long long wait_ns, void* stream);

/* ---- the launch for callers that may not allocate (no counterpart in the reference) ---------- */

/* uqb_decode_launch without caller-owned scratch: p->mo and p->ml are ignored and the split-KV partials go to a
 * 24 MiB array that is part of the library image (uqb_static_scratch_bytes() bytes; every device that loads the
 * library carries it until the process ends).  It is meant for hosts where this call cannot be preceded by a
 * device allocation: an engine that has already handed all device memory to its own pool, a plugin whose host
 * framework forbids cudaMalloc once inference has begun, a latency-critical thread that cannot take the
 * device-wide stall cudaMalloc/cudaFree may cause.  Queries, cache, page table, lengths and `out` are still the
 * caller's.  The function itself never allocates or frees (no cudaMalloc/cudaFree, no library allocator).
 *   - A call whose partials need more than the array (uqb_workspace_bytes(p) > uqb_static_scratch_bytes(), e.g.
 *     a very large B*Hkv*nsplit*rows*D) is refused with cudaErrorInvalidValue before anything is enqueued:
 *     lower p->nsplit or use uqb_decode_launch_ws.
 *   - The first call on each device looks the array's device address up (cudaGetSymbolAddress, with that device
 *     current); make that first call before any stream capture begins.
 *   - All calls on one device share the array and it keeps the previous call's partials.  Nothing in it has to
 *     start at zero (each call writes every slot it later reads), but two such calls that overlap on the GPU
 *     (different streams, no ordering between them) race on it: order them, or give one of them its own workspace. */
int uqb_decode_launch_static(const UQParams* p, int nwarps, int stages, void* stream);
size_t uqb_static_scratch_bytes(void);

/* ---- diagnostics (no counterpart in the reference) ------------------------------------------- */

/* Every device-side wait in this library is bounded; a wait that runs out records what it was
 * waiting for and the kernel returns.  Reads (and clears) the current device's record:
 * out4[0] = code (0 = none, 1 = a barrier wait of the attention kernel, 3 = a rank's flag in uqb_merge_wait_launch),
 * out4[1] = block, out4[2] = barrier id (code 3: the rank), out4[3] = tile (code 3: seq).  Synchronises the device.
 * When the code is not zero, the outputs of the calls since the last read are not answers (the kernel that gave up left
 * its results unwritten or partial): from the moment the code is set until this function has read and cleared it, every
 * decode call on the device writes NaN rows (bf16 outputs and fp32 partials alike), so the failure shows in the data
 * without a synchronising read; the launches themselves still return 0. */
int uqb_last_status(uint32_t out4[4]);
/* Which kernel the last uqb_decode_* call on this thread chose: 1 = CUDA-core path, 2 = tcgen05 path. */
int uqb_last_path(void);
/* Timing aid for benchmarks: while both are non-NULL (cudaEvent_t passed as void*), every uqb_decode_* call of
 * this thread records `before` and `after` on the launch stream around its attention kernel (not the combine). */
void uqb_debug_events(void* before, void* after);
/* Kernels launched by this library in this process (all threads). */
unsigned long long uqb_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
