// Shared device/host helpers of libuq_b200: the FP4 codec arithmetic, the partial-slot layout of the
// caller's scratch, and the status record that bounded waits write to.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "uq_params.h"

#define UQ_DEV __device__ __forceinline__

// ---- what the host adds to UQParams for one launch -------------------------------------------------
struct UQLaunch {
  const int32_t* pos_offset;  // [B] global position of shard-local key 0 (nullptr = 0)
  const int32_t* tree_mask;   // [B, K] draft-visibility bitmasks of a tree-masked verify (nullptr = chain: draft j sees drafts 0..j)
  int ns_eff;                 // partial slots actually used per (sequence, kv head): <= p.nsplit
  int G;                      // Hq / Hkv
  int rows;                   // K * G query rows per (sequence, kv head)
  int BM;                     // row stride of the scratch (uq_block_m)
  float sc2;                  // sm_scale * log2(e) (times k_ts for an NVFP4 cache): scores live in the exp2 domain
  float out_scale;            // multiplies the normalised output: 1, or v_ts for an NVFP4 cache
  // A call with more query rows than one launch takes is run as chunks of consecutive drafts: this launch holds drafts
  // k_first .. k_first + p.K - 1 of the caller's k_total (rows of q and out are indexed by the caller's draft number), and
  // the len_cut = k_total - k_first - p.K drafts after the chunk do not exist for it: chunk draft j then sees the keys
  // below (seq_len - len_cut) - p.K + j + 1 = seq_len - k_total + (k_first + j) + 1, the whole call's limit for that draft.
  // (A tree-masked call is chunked with len_cut = 0: bit t of tree_mask[b, k_first + j] decides about each of the k_total drafts.)
  int k_first, k_total, len_cut;
  unsigned int* status;       // this device's status record (4 words), see uq_report
  int expire_id;              // 0, or (for the test of the give-up path) 30: the softmax role never announces the query tile of a
                              // segment, so the wait on barrier 30 runs out after its full limit on an otherwise healthy kernel
};

// ---- where the combine of a context shard sends its packed partial (context split over peer memory) ----------------
// Every rank owns one exchange buffer, mapped on every other rank: [2 parities][world slots][slot_floats] floats, then
// [2][kMaxPeers] flag words, then one counter word.  A call with sequence number seq uses parity seq & 1: rank r stores its
// partial (o [rows, D], then lse2 [rows]) into slot r of every rank's buffer and then sets flag[parity][r] = seq there.
constexpr int kMaxPeers = 8;
struct UQPeerPush {
  float* slot[kMaxPeers];          // this rank's slot in every rank's buffer, parity applied (slot[rank] is the local one)
  unsigned int* flag[kMaxPeers];   // this rank's flag word in every rank's buffer, parity applied
  unsigned int* counter;           // local word counting the combine's finished blocks (zero between calls)
  size_t rows_total;               // rows of the whole call: the lse2 values follow rows_total * D floats of o
  int world;
  unsigned int seq;
  int raise;                       // 1: this launch is the call's last and raises the flags once its blocks are done
};
__host__ __device__ inline size_t uq_peer_slot_floats(size_t rows, int D) { return (rows * (size_t)(D + 1) + 3) / 4 * 4; }
__host__ __device__ inline size_t uq_peer_data_bytes(int world, size_t slot_floats) { return ((size_t)2 * world * slot_floats * sizeof(float) + 255) / 256 * 256; }
__host__ __device__ inline size_t uq_peer_total_bytes(int world, size_t slot_floats) { return uq_peer_data_bytes(world, slot_floats) + 2 * kMaxPeers * sizeof(unsigned int) + 64; }

// Scratch slot (b, hk, s): rows are r = j * G + g (draft j, head g of the group), row stride BM.
UQ_DEV size_t uq_slot(const UQParams& p, int b, int hk, int s) { return ((size_t)b * p.HKV + hk) * p.nsplit + s; }

// Sequence length as this launch sees it, and the row of q / out that belongs to (sequence b, this launch's draft j).
UQ_DEV int uq_seq_len(const UQParams& p, const UQLaunch& x, int b) { return p.seq_lens[b] - x.len_cut; }
UQ_DEV size_t uq_draft_row(const UQLaunch& x, int b, int j) { return (size_t)b * x.k_total + x.k_first + j; }

// Keys of sequence b held by this cache (whole context, or one shard of it).
UQ_DEV int uq_n_local(const UQParams& p, const UQLaunch& x, int b, int* off_out) {
  const int n = uq_seq_len(p, x, b);
  const int off = x.pos_offset ? x.pos_offset[b] : 0;
  *off_out = off;
  long long cap = (long long)p.max_pages * p.PAGE;
  long long nl = (long long)n - off;
  nl = nl < 0 ? 0 : (nl > cap ? cap : nl);
  return (int)nl;
}

// Does query (draft) j of sequence b see draft token t (the key at global position seq_len - K + t)?  Chain: t <= j.
// Tree (reference uqmt/tree.py:9-12): bit t of tree_mask[b, j].
UQ_DEV bool uq_sees_draft(const UQParams& p, const UQLaunch& x, int b, int j, int t) {
  return x.tree_mask ? ((static_cast<unsigned>(__ldg(x.tree_mask + (size_t)b * p.K + j)) >> t) & 1u) != 0u : t <= j;
}

// ---- status record ------------------------------------------------------------------------------------
// [0] code (0 none, 1 barrier wait ran out), [1] block, [2] barrier id, [3] tile.  First writer wins.
UQ_DEV void uq_report(unsigned int* status, unsigned code, unsigned bar, unsigned tile) {
  if (atomicCAS(&status[0], 0u, code) == 0u) {
    status[1] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    status[2] = bar;
    status[3] = tile;
  }
}

// ---- codec ------------------------------------------------------------------------------------------
// UE8M0 byte -> fp32 2^(s-127).  s = 0 gives the denormal 2^-127; s = 255 gives 2^128 = +inf in fp32
// (the reference's torch.exp2 does the same).
UQ_DEV float uq_scale_f32(unsigned s) {
  return s == 0 ? __int_as_float(0x00400000) : (s == 255 ? __int_as_float(0x7f800000) : __int_as_float((int)(s << 23)));
}

// NVFP4 block scale: e4m3fn byte -> fp32 (reference uqmt/quant.py:139-147 reads it with torch's float8_e4m3fn -> float).
// The low seven bits moved up by seven are an fp16 with the same mantissa and an exponent bias of 15 instead of 7, so one
// conversion and a multiply by 2^8 give the value, subnormals included; 0x7f / 0xff are the format's NaN.
UQ_DEV float uq_e4m3_f32(unsigned b) {
  const float v = __half2float(__ushort_as_half((unsigned short)(((b & 0x80u) << 8) | ((b & 0x7fu) << 7)))) * 256.f;
  return (b & 0x7fu) == 0x7fu ? __int_as_float(0x7fc00000) : v;
}

// e2m1 nibble -> exact fp32 value: (sign | code3 << 22) read as fp32 is value * 2^-126 (a denormal for
// 0.5, zero for 0), and one multiply by 2^126 normalises it without rounding.
UQ_DEV float uq_e2m1_f32(unsigned nib) {
  return __int_as_float((int)(((nib & 8u) << 28) | ((nib & 7u) << 22))) * 8.507059173023462e37f;
}
