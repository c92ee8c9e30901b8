// Byte permute between this library's cache (four arrays, one per stream: kc / vc [pages, Hkv, PAGE, D/2], ks / vs
// [pages, Hkv, PAGE, D/32]) and the slot layout of the upstream engines (one array [pages, PAGE, Hkv, slot] whose slot holds a
// token's K codes, K scale bytes, V codes, V scale bytes one after the other, padded to the allocator's slot size):
// the converter of the reference's compatibility notes (reference cuda/UPSTREAM_COMPAT.md:81-88, a torch permute / cat there).
// On the way out two representation details of the upstream encoder can be applied (reference cuda/UPSTREAM_COMPAT.md:93-95,
// cuda/compat/paper_rule_cpu_check.py:14-18): a code nibble 0x8 (minus zero) becomes 0x0, and a 32-channel group whose codes
// are all zero gets the scale byte 0, upstream's mark for an all-zero group.  Coming in needs nothing beyond the permute: both
// decode as code * 2^(byte - 127).
#include "uq_common.cuh"

namespace {

// One thread per (page, token, head, stream, group): the group's 16 code bytes and its scale byte.
template <bool kToUpstream>
__global__ void __launch_bounds__(256) uq_layout_kernel(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, uint8_t* aos, long long slots, int HKV,
                                                        int PAGE, int D, int slot_bytes, int flags) {
  const int G = D / 32;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= slots * 2 * G) return;
  const int g = (int)(i % G), stream = (int)((i / G) % 2);
  const long long slot = i / (2 * G);                       // (page, token, head) in the upstream order
  const int h = (int)(slot % HKV), t = (int)((slot / HKV) % PAGE);
  const long long page = slot / ((long long)HKV * PAGE);
  const long long row = (page * HKV + h) * PAGE + t;        // the same token in this library's order
  uint8_t* codes = (stream ? vc : kc) + row * (D / 2) + g * 16;
  uint8_t* scale = (stream ? vs : ks) + row * G + g;
  uint8_t* a_codes = aos + slot * slot_bytes + stream * (D / 2 + G) + g * 16;
  uint8_t* a_scale = aos + slot * slot_bytes + stream * (D / 2 + G) + D / 2 + g;
  if (kToUpstream) {
    uint4 c = *reinterpret_cast<const uint4*>(codes);
    uint32_t w[4] = {c.x, c.y, c.z, c.w};
    uint8_t sb = *scale;
    uint32_t any = 0;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const uint32_t mag = w[k] & 0x77777777u;
      any |= mag;
      if (flags & 1) {
        // bit 3 of a nibble survives only where the nibble's magnitude is not zero (magnitude + 7 carries into bit 3 iff it is >= 1)
        const uint32_t nz = (mag + 0x77777777u) & 0x88888888u;
        w[k] &= 0x77777777u | nz;
      }
    }
    if ((flags & 2) && any == 0) sb = 0;
    // slots are only byte-aligned in general (slot sizes such as D + 2G = 136 keep 8-byte alignment; a padded size may not)
    if ((reinterpret_cast<uintptr_t>(a_codes) & 15) == 0) *reinterpret_cast<uint4*>(a_codes) = make_uint4(w[0], w[1], w[2], w[3]);
    else {
#pragma unroll
      for (int k = 0; k < 16; k++) a_codes[k] = (uint8_t)(w[k >> 2] >> (8 * (k & 3)));
    }
    *a_scale = sb;
    if (stream == 0 && g == 0)
      for (int k = D + 2 * G; k < slot_bytes; k++) aos[slot * slot_bytes + k] = 0;   // the allocator's padding
  } else {
    uint32_t w[4];
    if ((reinterpret_cast<uintptr_t>(a_codes) & 15) == 0) {
      const uint4 c = *reinterpret_cast<const uint4*>(a_codes);
      w[0] = c.x; w[1] = c.y; w[2] = c.z; w[3] = c.w;
    } else {
#pragma unroll
      for (int k = 0; k < 4; k++) w[k] = (uint32_t)a_codes[4 * k] | ((uint32_t)a_codes[4 * k + 1] << 8) | ((uint32_t)a_codes[4 * k + 2] << 16) | ((uint32_t)a_codes[4 * k + 3] << 24);
    }
    *reinterpret_cast<uint4*>(codes) = make_uint4(w[0], w[1], w[2], w[3]);
    *scale = *a_scale;
  }
}

// The same permute staged through shared memory, for caches of any size that matters: a block owns 64 consecutive slots,
// which are one contiguous run of the upstream array that starts on a 64-byte boundary whatever the slot size, so that side
// is moved with whole 16-byte vectors by consecutive threads; the pieces of a slot (a stream's codes start 4, 2 or 1 bytes
// aligned inside it: 68 bytes into a slot of head_dim 128) are picked out of shared memory, where alignment costs nothing,
// and this library's side is written / read as 16-byte vectors of 64-byte code rows.  W = the widest access every piece
// of a slot is aligned to inside the staged run.
constexpr int kStagedSlots = 64;

// n / d for n < 2^32 with m = floor(2^32 / d) (d = 1 takes m = 2^32 - 1): the estimate is short by one at most
UQ_DEV uint32_t div_magic(uint32_t n, uint32_t d, uint32_t m, uint32_t& rem) {
  uint32_t q = __umulhi(n, m);
  uint32_t r = n - q * d;
  if (r >= d) { q++; r -= d; }
  rem = r;
  return q;
}

template <int W>
UQ_DEV uint4 stage_load16(const uint8_t* p) {
  uint32_t w[4];
  if (W == 4) {
#pragma unroll
    for (int k = 0; k < 4; k++) w[k] = *reinterpret_cast<const uint32_t*>(p + 4 * k);
  } else if (W == 2) {
#pragma unroll
    for (int k = 0; k < 4; k++) w[k] = (uint32_t) * reinterpret_cast<const uint16_t*>(p + 4 * k) | ((uint32_t) * reinterpret_cast<const uint16_t*>(p + 4 * k + 2) << 16);
  } else {
#pragma unroll
    for (int k = 0; k < 4; k++) w[k] = (uint32_t)p[4 * k] | ((uint32_t)p[4 * k + 1] << 8) | ((uint32_t)p[4 * k + 2] << 16) | ((uint32_t)p[4 * k + 3] << 24);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

template <int W>
UQ_DEV void stage_store16(uint8_t* p, uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  if (W == 4) {
#pragma unroll
    for (int k = 0; k < 4; k++) *reinterpret_cast<uint32_t*>(p + 4 * k) = w[k];
  } else if (W == 2) {
#pragma unroll
    for (int k = 0; k < 8; k++) *reinterpret_cast<uint16_t*>(p + 2 * k) = (uint16_t)(w[k >> 1] >> (16 * (k & 1)));
  } else {
#pragma unroll
    for (int k = 0; k < 16; k++) p[k] = (uint8_t)(w[k >> 2] >> (8 * (k & 3)));
  }
}

template <bool kToUpstream, int W>
__global__ void __launch_bounds__(256) uq_layout_staged_kernel(uint8_t* __restrict__ kc, uint8_t* __restrict__ ks, uint8_t* __restrict__ vc,
                                                               uint8_t* __restrict__ vs, uint8_t* __restrict__ aos, uint32_t slots, int HKV,
                                                               uint32_t hkv_magic, int PAGE, uint32_t page_magic, int D, int slot_bytes, int flags) {
  extern __shared__ __align__(16) uint8_t stage[];   // the block's slots as they lie in the upstream array
  const int G = D / 32, half = D / 2, stream_bytes = half + G;
  const int g_shift = D == 64 ? 1 : (D == 128 ? 2 : 3);
  const uint32_t s0 = blockIdx.x * (uint32_t)kStagedSlots;
  const int count = (int)min((uint32_t)kStagedSlots, slots - s0);
  const int bytes = count * slot_bytes, vecs = bytes >> 4;
  uint8_t* region = aos + (size_t)s0 * slot_bytes;
  if (!kToUpstream) {
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) reinterpret_cast<uint4*>(stage)[i] = __ldcs(reinterpret_cast<const uint4*>(region) + i);
    for (int i = (vecs << 4) + threadIdx.x; i < bytes; i += blockDim.x) stage[i] = region[i];   // (a last block of fewer slots may end inside a vector)
  } else if (slot_bytes > 2 * stream_bytes) {
    for (int i = threadIdx.x; i < (bytes + 15) >> 4; i += blockDim.x) reinterpret_cast<uint4*>(stage)[i] = make_uint4(0u, 0u, 0u, 0u);   // the allocator's padding
  }
  __syncthreads();
  for (int it = threadIdx.x; it < count * 2 * G; it += blockDim.x) {
    const int g = it & (G - 1), stream = (it >> g_shift) & 1, sl = it >> (g_shift + 1);
    uint32_t h, t;
    const uint32_t qs = div_magic(s0 + sl, (uint32_t)HKV, hkv_magic, h);   // slot = (page * PAGE + token) * HKV + head
    const uint32_t page = div_magic(qs, (uint32_t)PAGE, page_magic, t);
    const size_t row = ((size_t)page * HKV + h) * PAGE + t;                // the same token in this library's order
    uint8_t* st = stage + sl * slot_bytes + stream * stream_bytes;
    uint8_t* codes = (stream ? vc : kc) + row * half + g * 16;
    uint8_t* scale = (stream ? vs : ks) + row * G + g;
    if (kToUpstream) {
      const uint4 c = *reinterpret_cast<const uint4*>(codes);
      uint32_t w[4] = {c.x, c.y, c.z, c.w};
      uint8_t sb = *scale;
      uint32_t any = 0;
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const uint32_t mag = w[k] & 0x77777777u;
        any |= mag;
        if (flags & 1) w[k] &= 0x77777777u | ((mag + 0x77777777u) & 0x88888888u);   // bit 3 of a nibble survives only where its magnitude is not zero
      }
      if ((flags & 2) && any == 0) sb = 0;
      stage_store16<W>(st + g * 16, make_uint4(w[0], w[1], w[2], w[3]));
      st[half + g] = sb;
    } else {
      *reinterpret_cast<uint4*>(codes) = stage_load16<W>(st + g * 16);
      *scale = st[half + g];
    }
  }
  if (kToUpstream) {
    __syncthreads();
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) reinterpret_cast<uint4*>(region)[i] = reinterpret_cast<const uint4*>(stage)[i];
    for (int i = (vecs << 4) + threadIdx.x; i < bytes; i += blockDim.x) region[i] = stage[i];
  }
}

template <bool kToUpstream>
bool staged_launch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, uint8_t* aos, long long slots, int HKV, int PAGE, int D, int slot_bytes, int flags,
                   cudaStream_t s) {
  const size_t smem = (size_t)kStagedSlots * slot_bytes;
  if (slots >= (1ll << 31) || smem > 48 * 1024 || (reinterpret_cast<uintptr_t>(aos) & 15)) return false;
  const uint32_t hm = HKV == 1 ? 0xffffffffu : (uint32_t)((1ull << 32) / (unsigned)HKV), pm = PAGE == 1 ? 0xffffffffu : (uint32_t)((1ull << 32) / (unsigned)PAGE);
  const unsigned blocks = (unsigned)((slots + kStagedSlots - 1) / kStagedSlots);
  const int sb = D / 2 + D / 32;
  const int w = ((slot_bytes | sb) & 3) == 0 ? 4 : (((slot_bytes | sb) & 1) == 0 ? 2 : 1);
  if (w == 4) uq_layout_staged_kernel<kToUpstream, 4><<<blocks, 256, smem, s>>>(kc, ks, vc, vs, aos, (uint32_t)slots, HKV, hm, PAGE, pm, D, slot_bytes, flags);
  else if (w == 2) uq_layout_staged_kernel<kToUpstream, 2><<<blocks, 256, smem, s>>>(kc, ks, vc, vs, aos, (uint32_t)slots, HKV, hm, PAGE, pm, D, slot_bytes, flags);
  else uq_layout_staged_kernel<kToUpstream, 1><<<blocks, 256, smem, s>>>(kc, ks, vc, vs, aos, (uint32_t)slots, HKV, hm, PAGE, pm, D, slot_bytes, flags);
  return true;
}

}  // namespace

// dir 0: this library's arrays -> upstream slots (flags: 1 minus-zero codes become zero, 2 all-zero groups get scale byte 0);
// dir 1: upstream slots -> this library's arrays.
cudaError_t uq_layout_dispatch(int dir, uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, uint8_t* aos, long long pages, int HKV, int PAGE, int D,
                               int slot_bytes, int flags, cudaStream_t s) {
  if (!kc || !ks || !vc || !vs || !aos || pages < 0 || HKV < 1 || PAGE < 1 || !(D == 64 || D == 128 || D == 256)) return cudaErrorInvalidValue;
  if (slot_bytes < D + 2 * (D / 32) || (flags & ~3)) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc)) & 15) return cudaErrorInvalidValue;   // code rows are read and written as 16-byte vectors
  const long long slots = pages * PAGE * HKV, threads = slots * 2 * (D / 32);
  if (threads == 0) return cudaSuccess;
  if (dir == 0 ? staged_launch<true>(kc, ks, vc, vs, aos, slots, HKV, PAGE, D, slot_bytes, flags, s)
               : staged_launch<false>(kc, ks, vc, vs, aos, slots, HKV, PAGE, D, slot_bytes, 0, s))
    return cudaGetLastError();
  // (slot arrays that are not 16-byte aligned, slots beyond 768 bytes, more than 2^31 slots: one thread per group)
  const long long blocks = (threads + 255) / 256;
  if (blocks > 0x7fffffffll) return cudaErrorInvalidValue;
  if (dir == 0)
    uq_layout_kernel<true><<<(unsigned)blocks, 256, 0, s>>>(kc, ks, vc, vs, aos, slots, HKV, PAGE, D, slot_bytes, flags);
  else
    uq_layout_kernel<false><<<(unsigned)blocks, 256, 0, s>>>(kc, ks, vc, vs, aos, slots, HKV, PAGE, D, slot_bytes, 0);
  return cudaGetLastError();
}
