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
  const long long blocks = (threads + 255) / 256;
  if (blocks > 0x7fffffffll) return cudaErrorInvalidValue;
  if (dir == 0)
    uq_layout_kernel<true><<<(unsigned)blocks, 256, 0, s>>>(kc, ks, vc, vs, aos, slots, HKV, PAGE, D, slot_bytes, flags);
  else
    uq_layout_kernel<false><<<(unsigned)blocks, 256, 0, s>>>(kc, ks, vc, vs, aos, slots, HKV, PAGE, D, slot_bytes, 0);
  return cudaGetLastError();
}
