// Operator surface of the paged UltraQuant FP4 verify/decode attention, C++ linkage.
//
// This header declares, with the same names, argument meaning, struct layout and error behaviour,
// the host entry points of the reference's native op (reference cuda/uq_decode.h:11-43), so that code
// written against the reference (its torch binding cuda/uq_ext.cpp, its vector harness
// cuda/test_vectors.cu) links against libuq_b200.so unchanged.  The plain-C twin of every function,
// plus the entry points the reference does not have (append, context-split partials, merge, status),
// is in uq_b200.h.
//
// Cache layout (reference cuda/uq_decode.h:3-6):
//   kc, vc   uint8 [pages, Hkv, PAGE, D/2]    two e2m1 codes per byte, low nibble = even channel
//   ks, vs   uint8 [pages, Hkv, PAGE, D/32]   UE8M0: value 2^(s-127), every byte 0..255 is a scale
//   q        bf16  [B, K, Hq, D]
//   block_table int32 [B, max_pages]; seq_lens int32 [B], INCLUDING the K draft tokens, which already
//   sit in the cache at the last K positions.  Draft j attends to seq_len - K + j + 1 keys; a row
//   with no visible key is written as zeros.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

#include "uq_params.h"

// Rows of one (sequence, kv head) tile: max(16, pow2(K * pow2(Hq/Hkv))).  Scratch sizes use it.   (reference uq_decode.h:33)
int uq_block_m(int K, int HQ, int HKV);
// fp32 element counts of the caller-owned scratch: mo [B,Hkv,nsplit,BLOCK_M,D], ml [B,Hkv,nsplit,BLOCK_M].   (reference uq_decode.h:34-35)
size_t uq_mo_elems(const UQParams& p);
size_t uq_ml_elems(const UQParams& p);

// Asynchronous launch on `s`.  nwarps / stages / p.variant / p.mb are tuning hints of the reference's
// kernels: accepted, ignored.  p.nsplit (1..128) is the number of partial slots the scratch holds per
// (sequence, kv head); the kernels use at most that many.  Returns cudaErrorInvalidValue, before any
// work is enqueued, for a shape this library does not serve.   (reference uq_decode.h:37-39)
cudaError_t uq_decode_launch(const UQParams& p, int nwarps, int stages, cudaStream_t s);

// Same, with one caller-owned workspace (mo then ml, uq_workspace_bytes(p) bytes): no allocation, no
// synchronisation, no host read of device memory.   (reference uq_decode.h:40-42)
size_t uq_workspace_bytes(const UQParams& p);
cudaError_t uq_decode_launch_ws(UQParams p, void* workspace, int nwarps, int stages, cudaStream_t s);

// 1 only for a Hopper build on a Hopper device; this library is sm_100a only and returns 0.   (reference uq_decode.h:43)
int uq_has_sm90();
