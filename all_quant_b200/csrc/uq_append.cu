// KV append-quantize: encode new tokens to UltraQuant FP4 (e2m1 + UE8M0 per 32 channels) and scatter
// them into the paged cache.  Bit-exact with the reference encoder quantize_fp4
// (reference uqmt/attn.py:52-66) and its append hook (reference uqmt/vllm_adapter.py:48-59).
//
// One warp per (token, kv head, stream) where stream 0 = key, 1 = value; a lane owns four consecutive
// channels of each 128-channel slab, so a scale group is eight lanes and the group maximum is three
// shuffles.  HBM traffic is the input row plus D/2 + D/32 bytes out: the kernel is launch-latency
// sized for a decode step, so key and value go in one launch.
//
// Two options of the reference's configurable quantiser ride in the same kernel (flags):
//   1  the key row is rotated by the orthonormal Walsh-Hadamard transform over head_dim before it is encoded
//      (reference uqmt/quant.py:84-98 fwht; K and Q rotated alike leave q.k unchanged, V is not rotated): the same
//      butterfly order in fp32 (stages 1 and 2 in the lane's registers, 4..64 by shuffles, 128 across the two slabs of
//      head_dim 256), one division by (float)sqrt(D), and for a 16-bit input the rounding to that type which the
//      reference's function applies to its result.  uq_fwht_kernel is the same transform alone, for the queries.
//   2  the 'paper' scale rule E = round(log2(c * amax)) (half to even), values clipped at +-6
//      (reference uqmt/quant.py:52-60, quantize_on_write's rule argument :197-206) instead of ceil(log2(amax / 6)).
#include <cuda_fp8.h>

#include <type_traits>

#include "uq_common.cuh"

namespace {

template <typename T>
UQ_DEV float to_f32(T v);
template <>
UQ_DEV float to_f32<float>(float v) { return v; }
template <>
UQ_DEV float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
UQ_DEV float to_f32<__half>(__half v) { return __half2float(v); }
template <typename T>
UQ_DEV T from_f32(float v);
template <>
UQ_DEV float from_f32<float>(float v) { return v; }
template <>
UQ_DEV __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
UQ_DEV __half from_f32<__half>(float v) { return __float2half_rn(v); }

// four consecutive channels of a row as fp32: one 16-byte (fp32) or 8-byte (16-bit types) load when the row is aligned for it
template <typename T>
UQ_DEV void load4(const T* p, bool vec, float* out);
template <>
UQ_DEV void load4<float>(const float* p, bool vec, float* out) {
  if (vec) { const float4 v = __ldg(reinterpret_cast<const float4*>(p)); out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w; }
  else { for (int i = 0; i < 4; i++) out[i] = p[i]; }
}
template <>
UQ_DEV void load4<__nv_bfloat16>(const __nv_bfloat16* p, bool vec, float* out) {
  if (vec) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    out[0] = __uint_as_float(v.x << 16); out[1] = __uint_as_float(v.x & 0xffff0000u);
    out[2] = __uint_as_float(v.y << 16); out[3] = __uint_as_float(v.y & 0xffff0000u);
  } else { for (int i = 0; i < 4; i++) out[i] = __bfloat162float(p[i]); }
}
template <>
UQ_DEV void load4<__half>(const __half* p, bool vec, float* out) {
  if (vec) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
  } else { for (int i = 0; i < 4; i++) out[i] = __half2float(p[i]); }
}

constexpr int kRotateK = 1, kPaperRule = 2, kRouteBulk = 4;   // (flags & 8 names the per-row kernel: nothing to do for it here)

// Orthonormal Walsh-Hadamard transform of one row of D = 64 / 128 / 256 values held by a warp: lane l owns channels
// 128 s + 4 l .. + 3 of slab s (lanes 16.. hold zeros at D = 64).  Stage h pairs (i, i + h) -> (a + b, a - b), h ascending.
UQ_DEV void warp_fwht(float (&x)[2][4], int D, int lane) {
#pragma unroll
  for (int s = 0; s < 2; s++) {
    float a = x[s][0], b = x[s][1], c = x[s][2], d = x[s][3];
    x[s][0] = a + b; x[s][1] = a - b; x[s][2] = c + d; x[s][3] = c - d;            // h = 1
    a = x[s][0]; b = x[s][1]; c = x[s][2]; d = x[s][3];
    x[s][0] = a + c; x[s][2] = a - c; x[s][1] = b + d; x[s][3] = b - d;            // h = 2
  }
  const int within = D < 128 ? D : 128;
  for (int m = 1; 4 * m < within; m <<= 1) {                                       // h = 4 m
#pragma unroll
    for (int s = 0; s < 2; s++)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const float p = __shfl_xor_sync(0xffffffffu, x[s][i], m);
        x[s][i] = (lane & m) ? p - x[s][i] : x[s][i] + p;
      }
  }
  if (D == 256) {                                                                  // h = 128
#pragma unroll
    for (int i = 0; i < 4; i++) { const float a = x[0][i], b = x[1][i]; x[0][i] = a + b; x[1][i] = a - b; }
  }
  const float div = (float)sqrt((double)D);
#pragma unroll
  for (int s = 0; s < 2; s++)
#pragma unroll
    for (int i = 0; i < 4; i++) x[s][i] = __fdiv_rn(x[s][i], div);
}

// Scale exponent of a group: clamp(ceil(log2(max(amax, 1e-30) / 6)), -127, 127), evaluated as the
// reference evaluates it in fp32.  log2 is taken in double and rounded to fp32: that reproduces the
// correctly rounded fp32 log2 of the reference's CPU kernels, including the points a few ulp above a
// power of two where the fp32 result rounds down to the integer and ceil() does not step up.
// The double-precision log2 is slow on this part, and it only matters where the fp32 value lies within rounding
// distance of the point that decides the integer (an integer for ceil, a half for round): log2f (1 ulp, at most 2e-5 for
// |log2| <= 150) settles every other input, and the rare group closer than 1e-3 to a deciding point takes the double.
UQ_DEV int group_exponent(float amax, bool paper, float c) {
  amax = fmaxf(amax, 1e-30f);
  const float r = paper ? __fmul_rn(c, amax) : __fdiv_rn(amax, 6.0f);
  float t = log2f(r);
  const float frac = t - floorf(t);
  const bool near = paper ? fabsf(frac - 0.5f) < 1e-3f : (frac < 1e-3f || frac > 1.0f - 1e-3f);
  if (near) t = (float)log2((double)r);
  float e = paper ? rintf(t) : ceilf(t);   // rintf = torch.round: half to even
  e = fminf(fmaxf(e, -127.0f), 127.0f);
  return (int)e;
}

// e2m1 code of y = x / 2^e: nearest of {0,.5,1,1.5,2,3,4,6}, ties to the smaller magnitude (the
// reference's first-index argmin), sign bit from (y < 0) whatever the magnitude.
// The division by the power-of-two scale is a multiplication by its reciprocal 2^-e, which is exact for every e in
// [-127, 127] (2^127 and the denormal 2^-127 are both fp32 values): the same real quotient, so the same rounding.
UQ_DEV unsigned encode_e2m1(float x, float inv_scale) {
  float y = __fmul_rn(x, inv_scale);
  y = fminf(fmaxf(y, -6.0f), 6.0f);
  const float a = fabsf(y);
  unsigned c = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
  return c | (y < 0.0f ? 8u : 0u);
}

template <typename T>
__global__ void __launch_bounds__(128) uq_append_kernel(uint8_t* __restrict__ kc, uint8_t* __restrict__ ks, uint8_t* __restrict__ vc,
                                                        uint8_t* __restrict__ vs, const T* __restrict__ key, const T* __restrict__ value,
                                                        const int64_t* __restrict__ slots, int T_tok, int HKV, int D, int PAGE, int nstream,
                                                        int flags, float c) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int total = T_tok * HKV * nstream;
  if (warp >= total) return;
  const int stream = warp % nstream;
  const int h = (warp / nstream) % HKV;
  const int t = warp / (nstream * HKV);
  const int64_t slot = slots[t];
  if (slot < 0) return;
  int64_t page, off;
  if (slot <= 0x7fffffffll) { page = (uint32_t)slot / (uint32_t)PAGE; off = (uint32_t)slot % (uint32_t)PAGE; }   // the common case without a 64-bit division
  else { page = slot / PAGE; off = slot % PAGE; }
  const size_t row = ((size_t)page * HKV + h) * PAGE + off;
  const T* src = (stream == 0 ? key : value) + ((size_t)t * HKV + h) * D;
  uint8_t* codes = (stream == 0 ? kc : vc) + row * (D / 2);
  uint8_t* scales = (stream == 0 ? ks : vs) + row * (D / 32);
  const bool vec = ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value)) & 15) == 0;   // (rows are multiples of 64 channels)
  float xs[2][4];
#pragma unroll
  for (int sl = 0; sl < 2; sl++) {
    const int ch = sl * 128 + lane * 4;
    if (ch < D) load4<T>(src + ch, vec, xs[sl]);
    else xs[sl][0] = xs[sl][1] = xs[sl][2] = xs[sl][3] = 0.f;
  }
  if ((flags & kRotateK) && stream == 0) {
    warp_fwht(xs, D, lane);
#pragma unroll
    for (int sl = 0; sl < 2; sl++)
#pragma unroll
      for (int i = 0; i < 4; i++) xs[sl][i] = to_f32<T>(from_f32<T>(xs[sl][i]));   // the reference's transform returns its input's type
  }
  const bool paper = (flags & kPaperRule) != 0;
#pragma unroll
  for (int sl = 0; sl < 2; sl++) {
    const int ch = sl * 128 + lane * 4;
    if (sl * 128 >= D) break;
    const bool live = ch < D;   // D = 64: lanes 16..31 idle
    const float* x = xs[sl];
    float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
    for (int m = 1; m < 8; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    const int e = group_exponent(amax, paper, c);
    // 1 / 2^e as fp32; e = 127 gives the denormal 2^-127
    const float scale = e == 127 ? __int_as_float(0x00400000) : __int_as_float((127 - e) << 23);   // 2^-e
    if (live) {
      const unsigned c0 = encode_e2m1(x[0], scale), c1 = encode_e2m1(x[1], scale);
      const unsigned c2 = encode_e2m1(x[2], scale), c3 = encode_e2m1(x[3], scale);
      *reinterpret_cast<uint16_t*>(codes + ch / 2) = (uint16_t)(c0 | (c1 << 4) | (c2 << 8) | (c3 << 12));
      if ((lane & 7) == 0) scales[ch / 32] = (uint8_t)(e + 127);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The bulk form of the same encoder, for calls that write many tokens at once (a prompt's keys and values: hundreds of
// megabytes in, a quarter of that out).  The kernel above spends a warp's whole life on one 8-byte load per lane, which
// is right for a decode step (launch latency) and a tenth of the memory bandwidth for a prompt.  Here:
//   * a lane owns 8 consecutive channels (a piece: 16 bytes of a 16-bit input, 32 of fp32) of 8 (fp32: 4) runs of the
//     input, a warp-wide load is one contiguous 512-byte (1 KiB) run, and all of a thread's loads are issued before the
//     first is used: 4 KiB in flight per warp, 128 KiB per SM (with half of that the kernel waits on memory latency);
//   * a 32-channel group is four lanes: the group maximum takes two shuffles, and the four lanes share the work on the
//     scale exponents of their pieces (lane q computes those of pieces q, q + 4; a shuffle hands them round); the
//     row a piece belongs to (token, head, slot, page) is looked up once per row by one lane and handed round likewise;
//   * the codes come from the hardware conversion (cvt.rn.satfinite.e2m1x2.f32, two values per instruction) instead of
//     seven comparisons per value.  That conversion rounds a value half way between two code points to the even code,
//     the reference takes the smaller magnitude (first index of the minimum distance); the two differ at |y| = 0.75,
//     1.75 and 3.5 only.  A 16-bit input has at most 11 significant bits and y = x / 2^e keeps them, so multiplying by
//     the fp32 value just below 2^-e moves an exact half-way value one fp32 step down (where it rounds as the reference
//     does) and moves no other value across or onto a boundary; an fp32 input takes 2^-e itself and the three half-way
//     values are corrected by comparison.  The conversion keeps the sign of a negative value that rounds to zero, as
//     the reference does (sign bit = y < 0); adding +0 turns y = -0 (an input -0, or an underflow) into +0 first.
// Same bytes as the kernel above on every input (the tests run both on the same rows), rotated keys included (the transform
// runs across the D / 8 lanes of a row before anything else).  Not served here: inputs not aligned to 16 bytes, more than
// 2^31 pieces.
#ifndef UQ_BULK_THREADS
#define UQ_BULK_THREADS 128
#endif
constexpr long long kBulkMinRows = 4096;   // rows x streams from which a call goes to the bulk kernel

// One piece = 8 consecutive channels as loaded (16 bytes of a 16-bit type, two float4 of fp32).  A thread keeps its pieces
// in this form until it encodes them: 16-bit inputs stay packed (half the registers, so twice the pieces, and with them
// twice the bytes, in flight per thread), and their maximum is taken on the packed pairs.
template <typename T>
struct Piece {
  uint4 v;
  UQ_DEV void load(const T* p) { v = __ldcs(reinterpret_cast<const uint4*>(p)); }
  UQ_DEV void zero() { v = make_uint4(0u, 0u, 0u, 0u); }
  UQ_DEV float amax() const;
  UQ_DEV void values(float* x) const;
};
template <>
struct Piece<float> {
  float4 a, b;
  UQ_DEV void load(const float* p) { a = __ldcs(reinterpret_cast<const float4*>(p)); b = __ldcs(reinterpret_cast<const float4*>(p) + 1); }
  UQ_DEV void zero() { a = b = make_float4(0.f, 0.f, 0.f, 0.f); }
  UQ_DEV float amax() const {
    return fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))), fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
  }
  UQ_DEV void values(float* x) const { x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w; }
};
// (set(): eight fp32 values rounded to the piece's type, the rounding the reference's transform applies to its result)
template <typename T>
UQ_DEV void piece_set(Piece<T>& pc, const float* x);
template <>
UQ_DEV void piece_set<float>(Piece<float>& pc, const float* x) {
  pc.a = make_float4(x[0], x[1], x[2], x[3]);
  pc.b = make_float4(x[4], x[5], x[6], x[7]);
}
template <>
UQ_DEV void piece_set<__nv_bfloat16>(Piece<__nv_bfloat16>& pc, const float* x) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  pc.v = make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
UQ_DEV void piece_set<__half>(Piece<__half>& pc, const float* x) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const __half2 v = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  pc.v = make_uint4(w[0], w[1], w[2], w[3]);
}

// Orthonormal Walsh-Hadamard transform of rows of D channels whose lanes hold 8 consecutive channels each (D / 8 lanes per
// row, aligned): the butterfly order of warp_fwht (stage h pairs (i, i + h) -> (a + b, a - b), h ascending): h = 1, 2, 4
// inside the lane's eight values, h = 8 .. D / 2 across the row's lanes, then one division by (float)sqrt(D).
UQ_DEV void piece_fwht(float (&x)[8], int D, int lane) {
#pragma unroll
  for (int h = 1; h < 8; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
      if (!(i & h)) { const float a = x[i], b = x[i | h]; x[i] = a + b; x[i | h] = a - b; }
    }
  }
  for (int m = 1; 8 * m < D; m <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float p = __shfl_xor_sync(0xffffffffu, x[i], m);
      x[i] = (lane & m) ? p - x[i] : x[i] + p;
    }
  }
  const float div = (float)sqrt((double)D);
#pragma unroll
  for (int i = 0; i < 8; i++) x[i] = __fdiv_rn(x[i], div);
}

template <>
UQ_DEV float Piece<__nv_bfloat16>::amax() const {
  const uint32_t m0 = v.x & 0x7fff7fffu, m1 = v.y & 0x7fff7fffu, m2 = v.z & 0x7fff7fffu, m3 = v.w & 0x7fff7fffu;
  const __nv_bfloat162 m = __hmax2(__hmax2(*reinterpret_cast<const __nv_bfloat162*>(&m0), *reinterpret_cast<const __nv_bfloat162*>(&m1)),
                                   __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&m2), *reinterpret_cast<const __nv_bfloat162*>(&m3)));
  const uint32_t w = *reinterpret_cast<const uint32_t*>(&m);
  return fmaxf(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <>
UQ_DEV void Piece<__nv_bfloat16>::values(float* x) const {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; i++) { x[2 * i] = __uint_as_float(w[i] << 16); x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <>
UQ_DEV float Piece<__half>::amax() const {
  const uint32_t m0 = v.x & 0x7fff7fffu, m1 = v.y & 0x7fff7fffu, m2 = v.z & 0x7fff7fffu, m3 = v.w & 0x7fff7fffu;
  const __half2 m = __hmax2(__hmax2(*reinterpret_cast<const __half2*>(&m0), *reinterpret_cast<const __half2*>(&m1)),
                            __hmax2(*reinterpret_cast<const __half2*>(&m2), *reinterpret_cast<const __half2*>(&m3)));
  const float2 f = __half22float2(m);
  return fmaxf(f.x, f.y);
}
template <>
UQ_DEV void Piece<__half>::values(float* x) const {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; i++) { const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i])); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
}

template <typename T>
__host__ __device__ constexpr int bulk_pieces() { return sizeof(T) == 4 ? 4 : 8; }

// eight fp32 values -> eight e2m1 codes, value i in bits 4 i .. 4 i + 3 (round to nearest, half way to the even code, +-6 at most)
UQ_DEV uint32_t cvt_e2m1x8(const float* y) {
  uint32_t w;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}"
      : "=r"(w)
      : "f"(y[0]), "f"(y[1]), "f"(y[2]), "f"(y[3]), "f"(y[4]), "f"(y[5]), "f"(y[6]), "f"(y[7]));
  return w;
}

// n / d for n < 2^32 with m = floor(2^32 / d) (d >= 2; d = 1 takes m = 2^32 - 1): the estimate is short by one at most
UQ_DEV uint32_t div_magic(uint32_t n, uint32_t d, uint32_t m, uint32_t& rem) {
  uint32_t q = __umulhi(n, m);
  uint32_t r = n - q * d;
  if (r >= d) { q++; r -= d; }
  rem = r;
  return q;
}

template <typename T, bool kRot>
__global__ void __launch_bounds__(256) uq_append_bulk_kernel(uint8_t* __restrict__ kc, uint8_t* __restrict__ ks, uint8_t* __restrict__ vc,
                                                             uint8_t* __restrict__ vs, const T* __restrict__ key, const T* __restrict__ value,
                                                             const int64_t* __restrict__ slots, uint32_t np, int HKV, uint32_t hkv_magic, int D,
                                                             int PAGE, int page_shift, int paper, float c) {
  constexpr bool kExactTies = sizeof(T) == 4;   // fp32 inputs can sit anywhere: half-way values are corrected by comparison
  constexpr int NP = bulk_pieces<T>();          // pieces per thread: 128 bytes of input in flight
  const int stream = blockIdx.y;
  const T* __restrict__ src = stream ? value : key;
  uint8_t* __restrict__ codes = stream ? vc : kc;
  uint8_t* __restrict__ scales = stream ? vs : ks;
  const int lane = threadIdx.x & 31;
  const uint32_t wp0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * (32u * NP);   // the warp's first piece (8 channels)
  const uint32_t p0 = wp0 + lane;                                                            // this lane's first piece
  const int ppr_shift = D == 64 ? 3 : (D == 128 ? 4 : 5);   // pieces per row = D / 8
  Piece<T> pc[NP];
#pragma unroll
  for (int j = 0; j < NP; j++) {
    const uint32_t p = p0 + 32u * j;
    if (p < np) pc[j].load(src + (size_t)p * 8);
    else pc[j].zero();
  }
  // rotated keys: every row of the key stream goes through the transform first and is rounded to the input's type, as the
  // reference's function returns it; the pieces then hold the rotated row and everything below is unchanged
  if (kRot && stream == 0) {
#pragma unroll
    for (int j = 0; j < NP; j++) {
      float x[8];
      pc[j].values(x);
      piece_fwht(x, D, lane);
      piece_set<T>(pc[j], x);
    }
  }
  // Where the rows go: the warp's 32 * NP pieces are 4 .. 32 whole rows, lane L looks up row L (token, head, slot, page)
  // once and a piece fetches its row's answer by shuffle.  ~0 = no row (past the end, or a skipped token).
  unsigned long long my_off = ~0ull;   // byte offset of the row's codes in the cache
  {
    const uint32_t r = (wp0 >> ppr_shift) + lane;
    if (lane < ((32 * NP) >> ppr_shift) && r < (np >> ppr_shift)) {
      uint32_t h;
      const uint32_t t = div_magic(r, (uint32_t)HKV, hkv_magic, h);
      const int64_t slot = __ldg(slots + t);
      if (slot >= 0) {
        int64_t page, off;
        if (page_shift >= 0) { page = slot >> page_shift; off = slot & ((1ll << page_shift) - 1); }
        else if (slot <= 0x7fffffffll) { page = (uint32_t)slot / (uint32_t)PAGE; off = (uint32_t)slot % (uint32_t)PAGE; }
        else { page = slot / PAGE; off = slot % PAGE; }
        my_off = (((unsigned long long)page * HKV + h) * PAGE + off) * (unsigned)(D / 2);
      }
    }
  }
  // group maxima (a group = the four lanes of a piece), and the scales: lane q of a group computes the exponents of pieces
  // q, q + 4, ... and from them the multipliers 2^-e (e = 127 gives the denormal 2^-127; a 16-bit input takes the fp32
  // value just below 2^-e); the encoding loop fetches each piece's multiplier by shuffle and reads the scale byte off it
  const int q = lane & 3;
  constexpr uint32_t kBelow = kExactTies ? 0u : 1u;
  uint32_t inv_mine[NP / 4];
  // y = -0 must become +0 (the reference's sign bit is y < 0).  x * s + (+0) does that for an input -0 at no cost, but a
  // negative product too small for fp32 still rounds to -0: possible only when the smallest non-zero magnitude of the
  // 16-bit input type (2^-133 bf16, 2^-24 fp16) times 2^-e does not exceed 2^-150 (2^-150 itself is half way between 0
  // and the smallest denormal and rounds to zero), i.e. for bf16 groups whose maximum is beyond 6 * 2^16; a warp that
  // holds such a group, and every warp of an fp32 input, adds +0 after the multiplication instead
  constexpr int kTiny = std::is_same<T, __nv_bfloat16>::value ? -133 : -24;
  bool tiny = sizeof(T) == 4;
#pragma unroll
  for (int r = 0; r < NP / 4; r++) {
    float am = 0.f;
#pragma unroll
    for (int jj = 0; jj < 4; jj++) {
      float a = pc[4 * r + jj].amax();
      a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
      a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
      if (q == jj) am = a;
    }
    const int e = group_exponent(am, paper != 0, c);
    inv_mine[r] = (e == 127 ? 0x00400000u : (uint32_t)(127 - e) << 23) - kBelow;
    tiny |= kTiny - e <= -150;
  }
  const bool add_zero = sizeof(T) == 4 || __any_sync(0xffffffffu, tiny);
  auto encode = [&](auto add_zero_c) {
#pragma unroll
    for (int j = 0; j < NP; j++) {
      const uint32_t inv = __shfl_sync(0xffffffffu, inv_mine[j >> 2], (lane & ~3) | (j & 3));
      const unsigned long long off = __shfl_sync(0xffffffffu, my_off, (32 * j + lane) >> ppr_shift);
      const float s = __uint_as_float(inv);
      float x[8], y[8];
      pc[j].values(x);
#pragma unroll
      for (int i = 0; i < 8; i++) y[i] = decltype(add_zero_c)::value ? __fadd_rn(__fmul_rn(x[i], s), 0.0f) : __fmaf_rn(x[i], s, 0.0f);
      uint32_t w = cvt_e2m1x8(y);
      if (kExactTies) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float a = fabsf(y[i]);
          if (a == 0.75f || a == 1.75f || a == 3.5f) w -= 1u << (4 * i);   // half way and rounded up to the even code: the reference stays below
        }
      }
      if (off != ~0ull) {
        const uint32_t piece = (p0 + 32u * j) & ((1u << ppr_shift) - 1u);
        *reinterpret_cast<uint32_t*>(codes + off + piece * 4) = w;
        // scale byte e + 127 = 254 - (exponent field of 2^-e), which is 0 for the denormal 2^-127; a row's scale bytes
        // start at 1/16 of its codes' offset
        if (q == 0) scales[(off >> 4) + (piece >> 2)] = (uint8_t)(254u - ((inv + kBelow) >> 23));
      }
    }
  };
  if (add_zero) encode(std::true_type{});
  else encode(std::false_type{});
}

// the bulk kernel serves: pointers aligned for the vector loads, piece count within 32 bits
template <typename T>
bool bulk_launch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const T* key, const T* value, const int64_t* slots, int T_tok, int HKV,
                 int D, int PAGE, int nstream, int flags, float c, cudaStream_t s) {
  const unsigned long long np = (unsigned long long)T_tok * HKV * (D / 8);
  const uintptr_t al = 15;
  if (np >= (1ull << 31) || ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value)) & al)) return false;
  const uint32_t magic = HKV == 1 ? 0xffffffffu : (uint32_t)((1ull << 32) / (unsigned)HKV);
  int shift = -1;
  if ((PAGE & (PAGE - 1)) == 0) { shift = 0; while ((1 << shift) < PAGE) shift++; }
  const unsigned per_block = (UQ_BULK_THREADS / 32u) * 32u * bulk_pieces<T>();
  const dim3 grid((unsigned)((np + per_block - 1) / per_block), (unsigned)nstream);
  if (flags & kRotateK)
    uq_append_bulk_kernel<T, true><<<grid, UQ_BULK_THREADS, 0, s>>>(kc, ks, vc, vs, key, value, slots, (uint32_t)np, HKV, magic, D, PAGE, shift, (flags & kPaperRule) ? 1 : 0, c);
  else
    uq_append_bulk_kernel<T, false><<<grid, UQ_BULK_THREADS, 0, s>>>(kc, ks, vc, vs, key, value, slots, (uint32_t)np, HKV, magic, D, PAGE, shift, (flags & kPaperRule) ? 1 : 0, c);
  return true;
}

// NVFP4 append (reference uqmt/quant.py:125-136 quantize_nvfp4 with the tensor scale given; the byte view and the paged
// cache of uqmt/nvfp4.py:200-254): a block is 16 channels = four lanes; its scale is e4m3fn(clamp(amax / 6 / ts, 2^-9, 448))
// (two fp32 divisions, the hardware's round-to-nearest-even conversion), the codes are the nearest e2m1 values to
// x / (float(scale) * ts) clipped at +-6.  Same warp layout as the UltraQuant kernel; scale bytes [.., D/16].
template <typename T>
__global__ void __launch_bounds__(128) uq_append_nvfp4_kernel(uint8_t* __restrict__ kc, uint8_t* __restrict__ ks, uint8_t* __restrict__ vc,
                                                              uint8_t* __restrict__ vs, const T* __restrict__ key, const T* __restrict__ value,
                                                              const int64_t* __restrict__ slots, int T_tok, int HKV, int D, int PAGE, float k_ts,
                                                              float v_ts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T_tok * HKV * 2) return;
  const int stream = warp & 1;
  const int h = (warp >> 1) % HKV;
  const int t = warp / (2 * HKV);
  const int64_t slot = slots[t];
  if (slot < 0) return;
  const int64_t page = slot / PAGE, off = slot % PAGE;
  const size_t row = ((size_t)page * HKV + h) * PAGE + off;
  const T* src = (stream == 0 ? key : value) + ((size_t)t * HKV + h) * D;
  uint8_t* codes = (stream == 0 ? kc : vc) + row * (D / 2);
  uint8_t* scales = (stream == 0 ? ks : vs) + row * (D / 16);
  const float ts = stream == 0 ? k_ts : v_ts;
  const bool vec = ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value)) & 15) == 0;
  for (int base = 0; base < D; base += 128) {
    const int ch = base + lane * 4;
    const bool live = ch < D;   // D = 64: lanes 16..31 idle
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) load4<T>(src + ch, vec, x);
    float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float r = __fdiv_rn(__fdiv_rn(amax, 6.0f), ts);
    r = fminf(fmaxf(r, 0.001953125f), 448.0f);   // (NaN inputs are not reproduced: here they vanish from the maximum, torch carries them into the scale)
    const unsigned sb = (unsigned)__nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
    const float sf = __fmul_rn(uq_e4m3_f32(sb), ts);
    if (live) {
      unsigned c[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        float y = __fdiv_rn(x[i], sf);
        y = fminf(fmaxf(y, -6.0f), 6.0f);
        const float a = fabsf(y);
        c[i] = ((a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f)) | (y < 0.0f ? 8u : 0u);
      }
      *reinterpret_cast<uint16_t*>(codes + ch / 2) = (uint16_t)(c[0] | (c[1] << 4) | (c[2] << 8) | (c[3] << 12));
      if ((lane & 3) == 0) scales[ch / 16] = (uint8_t)sb;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The bulk form of the NVFP4 append: the layout of uq_append_bulk_kernel (pieces of 8 channels, a row lookup per lane), a
// block of 16 channels = two lanes.  The reference divides every value by the block's scale (float(e4m3 byte) * ts, not a
// power of two); an fp32 division is ten instructions, and the code only depends on which side of seven boundaries the
// quotient falls.  So the quotient is bracketed instead: y_lo = x * r_lo and y_hi = x * r_hi with r_lo / r_hi a fast
// reciprocal of the scale times (1 -+ 2^-21), which lie strictly below / above the reference's rounded quotient in
// magnitude (the reciprocal is good to 2^-22, the factor is two to four fp32 steps).  Both go through the hardware
// conversion; where the two codes of a value agree, no boundary lies inside its bracket and the code is the reference's
// whatever the tie rule of the conversion (a quotient exactly on a boundary has y_lo below and y_hi above it, so the two
// differ).  Where they differ the value is decided exactly: the reference's rounded quotient exceeds the boundary b iff
// |x| / sf > b + ulp(b) / 2 (b has an even mantissa, so a quotient half way rounds to b itself), i.e. iff
// |x| > (b + ulp(b) / 2) * sf, a product that is exact in double precision (25 x 24 bits); its sign bit is set iff x < 0 and
// the quotient does not round to zero, |x| > 2^-150 * sf.  That happens often enough to matter with 16-bit inputs (a value
// of 8 significant bits over a scale of 4 lands exactly on a boundary about once in a hundred), so the decision is a short
// loop over the differing codes of a lane, not a second pass over the piece.  Blocks whose scale is too small or large
// for the fast reciprocal (below 1e-30, above 1e30; for bf16 above 2^12, where a product could underflow to -0) are
// encoded with the division and the comparisons of the per-row kernel.  +0 is added to both products of an fp32 input
// (x * r + 0 for a 16-bit one), so a quotient that the reference rounds to -0 ("not < 0") and a bracket end that keeps a
// negative denormal disagree and are decided as above.
__constant__ double kNvBoundary[8] = {   // b + ulp_fp32(b) / 2 for the boundary above magnitude code c
    0.25 + 0x1p-26, 0.75 + 0x1p-25, 1.25 + 0x1p-24, 1.75 + 0x1p-24, 2.5 + 0x1p-23, 3.5 + 0x1p-23, 5.0 + 0x1p-22, 1e300};

__device__ __noinline__ uint32_t encode8_exact_nvfp4(const float* x, float sf) {
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    float y = __fdiv_rn(x[i], sf);
    y = fminf(fmaxf(y, -6.0f), 6.0f);
    const float a = fabsf(y);
    const uint32_t c = ((a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f)) | (y < 0.0f ? 8u : 0u);
    w |= c << (4 * i);
  }
  return w;
}

template <typename T>
__global__ void __launch_bounds__(256) uq_append_nvfp4_bulk_kernel(uint8_t* __restrict__ kc, uint8_t* __restrict__ ks, uint8_t* __restrict__ vc,
                                                                   uint8_t* __restrict__ vs, const T* __restrict__ key, const T* __restrict__ value,
                                                                   const int64_t* __restrict__ slots, uint32_t np, int HKV, uint32_t hkv_magic, int D,
                                                                   int PAGE, int page_shift, float k_ts, float v_ts) {
  constexpr int NP = bulk_pieces<T>();
  constexpr bool kAddZero = sizeof(T) == 4;   // fp32 inputs: any product can underflow, +0 is added after the multiplication
  // a 16-bit input's smallest non-zero magnitude (2^-133 bf16, 2^-24 fp16) times the reciprocal stays a normal number
  // as long as the scale is below this; beyond it the piece takes the exact path
  constexpr float kSfMax = std::is_same<T, __nv_bfloat16>::value ? 4096.0f /* 2^12 */ : 1e30f;
  const int stream = blockIdx.y;
  const T* __restrict__ src = stream ? value : key;
  uint8_t* __restrict__ codes = stream ? vc : kc;
  uint8_t* __restrict__ scales = stream ? vs : ks;
  const float ts = stream ? v_ts : k_ts;
  const int lane = threadIdx.x & 31;
  const uint32_t wp0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * (32u * NP);
  const uint32_t p0 = wp0 + lane;
  const int ppr_shift = D == 64 ? 3 : (D == 128 ? 4 : 5);
  Piece<T> pc[NP];
#pragma unroll
  for (int j = 0; j < NP; j++) {
    const uint32_t p = p0 + 32u * j;
    if (p < np) pc[j].load(src + (size_t)p * 8);
    else pc[j].zero();
  }
  unsigned long long my_off = ~0ull;   // byte offset of the row's codes in the cache
  {
    const uint32_t r = (wp0 >> ppr_shift) + lane;
    if (lane < ((32 * NP) >> ppr_shift) && r < (np >> ppr_shift)) {
      uint32_t h;
      const uint32_t t = div_magic(r, (uint32_t)HKV, hkv_magic, h);
      const int64_t slot = __ldg(slots + t);
      if (slot >= 0) {
        int64_t page, off;
        if (page_shift >= 0) { page = slot >> page_shift; off = slot & ((1ll << page_shift) - 1); }
        else if (slot <= 0x7fffffffll) { page = (uint32_t)slot / (uint32_t)PAGE; off = (uint32_t)slot % (uint32_t)PAGE; }
        else { page = slot / PAGE; off = slot % PAGE; }
        my_off = (((unsigned long long)page * HKV + h) * PAGE + off) * (unsigned)(D / 2);
      }
    }
  }
  // block maxima (a block = the two lanes of a piece); the two lanes share the work on the scales: the even lane takes
  // the even pieces, the odd lane the odd ones, a shuffle hands the results round
  const int par = lane & 1;
  float r_lo[NP / 2], r_hi[NP / 2], sf_m[NP / 2];
  uint32_t sb_m[NP / 2];   // scale byte | 0x100 when the fast path does not serve this block
#pragma unroll
  for (int i = 0; i < NP / 2; i++) {
    float a0 = pc[2 * i].amax(), a1 = pc[2 * i + 1].amax();
    a0 = fmaxf(a0, __shfl_xor_sync(0xffffffffu, a0, 1));
    a1 = fmaxf(a1, __shfl_xor_sync(0xffffffffu, a1, 1));
    const float amax = par ? a1 : a0;
    float r = __fdiv_rn(__fdiv_rn(amax, 6.0f), ts);
    r = fminf(fmaxf(r, 0.001953125f), 448.0f);   // (NaN inputs are not reproduced: here they vanish from the maximum, torch carries them into the scale)
    const uint32_t sb = (uint32_t)__nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
    const float sf = __fmul_rn(uq_e4m3_f32(sb), ts);
    float rc;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rc) : "f"(sf));
    const bool fast = sf > 1e-30f && sf < kSfMax;   // (also false for a scale that is not a number)
    r_lo[i] = __fmul_rn(rc, 0x1.fffffp-1f);    // 1 - 2^-21
    r_hi[i] = __fmul_rn(rc, 0x1.000008p+0f);   // 1 + 2^-21
    sf_m[i] = sf;
    sb_m[i] = sb | (fast ? 0u : 0x100u);
  }
#pragma unroll
  for (int j = 0; j < NP; j++) {
    const int from = (lane & ~1) | (j & 1);
    const float lo = __shfl_sync(0xffffffffu, r_lo[j >> 1], from), hi = __shfl_sync(0xffffffffu, r_hi[j >> 1], from);
    const uint32_t sbf = __shfl_sync(0xffffffffu, sb_m[j >> 1], from);
    const float sf = __shfl_sync(0xffffffffu, sf_m[j >> 1], from);
    const unsigned long long off = __shfl_sync(0xffffffffu, my_off, (32 * j + lane) >> ppr_shift);
    float x[8], y[8];
    pc[j].values(x);
#pragma unroll
    for (int i = 0; i < 8; i++) y[i] = kAddZero ? __fadd_rn(__fmul_rn(x[i], lo), 0.0f) : __fmaf_rn(x[i], lo, 0.0f);
    uint32_t w = cvt_e2m1x8(y);
#pragma unroll
    for (int i = 0; i < 8; i++) y[i] = kAddZero ? __fadd_rn(__fmul_rn(x[i], hi), 0.0f) : __fmaf_rn(x[i], hi, 0.0f);
    const uint32_t w_hi = cvt_e2m1x8(y);
    if (sbf & 0x100u) {
      w = encode8_exact_nvfp4(x, sf);
    } else {
      uint32_t d = w ^ w_hi;
      while (d) {   // the values whose bracket holds a boundary (or the edge of zero): decided exactly, one at a time
        const int sh = (__ffs(d) - 1) & ~3, idx = sh >> 2;
        const float xv = idx < 4 ? (idx < 2 ? (idx == 0 ? x[0] : x[1]) : (idx == 2 ? x[2] : x[3]))
                                 : (idx < 6 ? (idx == 4 ? x[4] : x[5]) : (idx == 6 ? x[6] : x[7]));
        const uint32_t c = (w >> sh) & 7u, c_hi = (w_hi >> sh) & 7u;
        const double ax = (double)fabsf(xv), sfd = (double)sf;
        const uint32_t mag = c + ((c_hi != c && ax > kNvBoundary[c] * sfd) ? 1u : 0u);
        const uint32_t neg = (xv < 0.0f && ax > sfd * 0x1p-150) ? 8u : 0u;
        w = (w & ~(0xFu << sh)) | ((mag | neg) << sh);
        d &= ~(0xFu << sh);
      }
    }
    if (off != ~0ull) {
      const uint32_t piece = (p0 + 32u * j) & ((1u << ppr_shift) - 1u);
      *reinterpret_cast<uint32_t*>(codes + off + piece * 4) = w;
      if (par == 0) scales[(off >> 3) + (piece >> 1)] = (uint8_t)sbf;   // (a row's scale bytes start at 1/8 of its codes' offset)
    }
  }
}

template <typename T>
bool bulk_nvfp4_launch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const T* key, const T* value, const int64_t* slots, int T_tok, int HKV,
                       int D, int PAGE, float k_ts, float v_ts, cudaStream_t s) {
  const unsigned long long np = (unsigned long long)T_tok * HKV * (D / 8);
  if (np >= (1ull << 31) || ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value)) & 15)) return false;
  const uint32_t magic = HKV == 1 ? 0xffffffffu : (uint32_t)((1ull << 32) / (unsigned)HKV);
  int shift = -1;
  if ((PAGE & (PAGE - 1)) == 0) { shift = 0; while ((1 << shift) < PAGE) shift++; }
  const unsigned per_block = (UQ_BULK_THREADS / 32u) * 32u * bulk_pieces<T>();
  const dim3 grid((unsigned)((np + per_block - 1) / per_block), 2u);
  uq_append_nvfp4_bulk_kernel<T><<<grid, UQ_BULK_THREADS, 0, s>>>(kc, ks, vc, vs, key, value, slots, (uint32_t)np, HKV, magic, D, PAGE, shift, k_ts, v_ts);
  return true;
}

// The transform alone (the queries of a cache whose keys were rotated): one warp per row, out may be x.
template <typename T>
__global__ void __launch_bounds__(128) uq_fwht_kernel(const T* __restrict__ x, T* __restrict__ out, long long rows, int D) {
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float xs[2][4];
#pragma unroll
  for (int sl = 0; sl < 2; sl++) {
    const int ch = sl * 128 + lane * 4;
#pragma unroll
    for (int i = 0; i < 4; i++) xs[sl][i] = ch < D ? to_f32<T>(x[row * D + ch + i]) : 0.f;
  }
  warp_fwht(xs, D, lane);
#pragma unroll
  for (int sl = 0; sl < 2; sl++) {
    const int ch = sl * 128 + lane * 4;
#pragma unroll
    for (int i = 0; i < 4; i++)
      if (ch < D) out[row * D + ch + i] = from_f32<T>(xs[sl][i]);
  }
}

}  // namespace

cudaError_t uq_fwht_dispatch(const void* x, void* out, long long rows, int D, int dtype, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (!x || !out || rows < 0 || !(D == 64 || D == 128 || D == 256) || dtype < 0 || dtype > 2) return cudaErrorInvalidValue;
  const long long blocks = (rows + 3) / 4;
  if (blocks > 0x7fffffffll) return cudaErrorInvalidValue;
  switch (dtype) {
    case 0: uq_fwht_kernel<float><<<(int)blocks, 128, 0, s>>>((const float*)x, (float*)out, rows, D); break;
    case 1: uq_fwht_kernel<__nv_bfloat16><<<(int)blocks, 128, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, rows, D); break;
    default: uq_fwht_kernel<__half><<<(int)blocks, 128, 0, s>>>((const __half*)x, (__half*)out, rows, D); break;
  }
  return cudaGetLastError();
}

// route: 0 by the size of the call, 4 the bulk kernel, 8 the per-row kernel (as the flags of uq_append_dispatch)
cudaError_t uq_append_nvfp4_dispatch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const void* key, const void* value,
                                     const int64_t* slots, int T, int HKV, int D, int PAGE, int dtype, float k_ts, float v_ts, cudaStream_t s, int route) {
  if (T == 0) return cudaSuccess;
  if (!kc || !ks || !vc || !vs || !key || !value || !slots) return cudaErrorInvalidValue;
  if (!(D == 64 || D == 128 || D == 256) || PAGE <= 0 || HKV <= 0 || T < 0 || dtype < 0 || dtype > 2) return cudaErrorInvalidValue;
  if (!(k_ts > 0.f) || !(v_ts > 0.f) || (route != 0 && route != 4 && route != 8)) return cudaErrorInvalidValue;
  const long long warps = (long long)T * HKV * 2;
  if (route == kRouteBulk || (route == 0 && warps >= kBulkMinRows)) {
    bool done = false;
    switch (dtype) {
      case 0: done = bulk_nvfp4_launch<float>(kc, ks, vc, vs, (const float*)key, (const float*)value, slots, T, HKV, D, PAGE, k_ts, v_ts, s); break;
      case 1: done = bulk_nvfp4_launch<__nv_bfloat16>(kc, ks, vc, vs, (const __nv_bfloat16*)key, (const __nv_bfloat16*)value, slots, T, HKV, D, PAGE, k_ts, v_ts, s); break;
      default: done = bulk_nvfp4_launch<__half>(kc, ks, vc, vs, (const __half*)key, (const __half*)value, slots, T, HKV, D, PAGE, k_ts, v_ts, s); break;
    }
    if (done) return cudaGetLastError();
    if (route == kRouteBulk) return cudaErrorInvalidValue;
  }
  const int blocks = (int)((warps + 3) / 4);
  switch (dtype) {
    case 0: uq_append_nvfp4_kernel<float><<<blocks, 128, 0, s>>>(kc, ks, vc, vs, (const float*)key, (const float*)value, slots, T, HKV, D, PAGE, k_ts, v_ts); break;
    case 1: uq_append_nvfp4_kernel<__nv_bfloat16><<<blocks, 128, 0, s>>>(kc, ks, vc, vs, (const __nv_bfloat16*)key, (const __nv_bfloat16*)value, slots, T, HKV, D, PAGE, k_ts, v_ts); break;
    default: uq_append_nvfp4_kernel<__half><<<blocks, 128, 0, s>>>(kc, ks, vc, vs, (const __half*)key, (const __half*)value, slots, T, HKV, D, PAGE, k_ts, v_ts); break;
  }
  return cudaGetLastError();
}

// dtype: 0 fp32, 1 bf16, 2 fp16.  value/vc/vs may be null (single-stream form).  flags: 1 rotate the keys, 2 'paper' rule with constant c,
// 4 / 8 take the bulk / the per-row kernel whatever the size of the call (neither: by size).
cudaError_t uq_append_dispatch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const void* key, const void* value,
                               const int64_t* slots, int T, int HKV, int D, int PAGE, int dtype, cudaStream_t s, int flags, float c) {
  if (T == 0) return cudaSuccess;   // nothing to write; empty tensors may come with null pointers
  if (!kc || !ks || !key || !slots) return cudaErrorInvalidValue;
  const bool two = value != nullptr;
  if (two && (!vc || !vs)) return cudaErrorInvalidValue;
  if (!(D == 64 || D == 128 || D == 256) || PAGE <= 0 || HKV <= 0 || T < 0 || dtype < 0 || dtype > 2) return cudaErrorInvalidValue;
  if ((flags & ~15) || (flags & 12) == 12 || ((flags & 2) && !(c > 0.f))) return cudaErrorInvalidValue;
  const int route = flags & 12;
  flags &= 3;
  const int nstream = two ? 2 : 1;
  const long long warps = (long long)T * HKV * nstream;
  // many rows: the bulk kernel (flags & 4 sends the call there whatever its size, flags & 8 keeps it here: the tests
  // compare the two on the same rows)
  if (route == kRouteBulk || (route == 0 && warps >= kBulkMinRows)) {
    bool done = false;
    switch (dtype) {
      case 0: done = bulk_launch<float>(kc, ks, vc, vs, (const float*)key, (const float*)value, slots, T, HKV, D, PAGE, nstream, flags, c, s); break;
      case 1: done = bulk_launch<__nv_bfloat16>(kc, ks, vc, vs, (const __nv_bfloat16*)key, (const __nv_bfloat16*)value, slots, T, HKV, D, PAGE, nstream, flags, c, s); break;
      default: done = bulk_launch<__half>(kc, ks, vc, vs, (const __half*)key, (const __half*)value, slots, T, HKV, D, PAGE, nstream, flags, c, s); break;
    }
    if (done) return cudaGetLastError();
    if (route == kRouteBulk) return cudaErrorInvalidValue;   // asked for by name and not served (alignment, size)
  }
  const int blocks = (int)((warps + 3) / 4);
  switch (dtype) {
    case 0: uq_append_kernel<float><<<blocks, 128, 0, s>>>(kc, ks, vc, vs, (const float*)key, (const float*)value, slots, T, HKV, D, PAGE, nstream, flags, c); break;
    case 1: uq_append_kernel<__nv_bfloat16><<<blocks, 128, 0, s>>>(kc, ks, vc, vs, (const __nv_bfloat16*)key, (const __nv_bfloat16*)value, slots, T, HKV, D, PAGE, nstream, flags, c); break;
    default: uq_append_kernel<__half><<<blocks, 128, 0, s>>>(kc, ks, vc, vs, (const __half*)key, (const __half*)value, slots, T, HKV, D, PAGE, nstream, flags, c); break;
  }
  return cudaGetLastError();
}
