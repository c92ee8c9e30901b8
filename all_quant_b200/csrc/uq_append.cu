// KV append-quantize: encode new tokens to UltraQuant FP4 (e2m1 + UE8M0 per 32 channels) and scatter
// them into the paged cache.  Bit-exact with the reference encoder quantize_fp4
// (reference uqmt/attn.py:52-66) and its append hook (reference uqmt/vllm_adapter.py:48-59).
//
// One warp per (token, kv head, stream) where stream 0 = key, 1 = value; a lane owns four consecutive
// channels of each 128-channel slab, so a scale group is eight lanes and the group maximum is three
// shuffles.  HBM traffic is the input row plus D/2 + D/32 bytes out: the kernel is launch-latency
// sized for a decode step, so key and value go in one launch.
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

// Scale exponent of a group: clamp(ceil(log2(max(amax, 1e-30) / 6)), -127, 127), evaluated as the
// reference evaluates it in fp32.  log2 is taken in double and rounded to fp32: that reproduces the
// correctly rounded fp32 log2 of the reference's CPU kernels, including the points a few ulp above a
// power of two where the fp32 result rounds down to the integer and ceil() does not step up.
UQ_DEV int group_exponent(float amax) {
  amax = fmaxf(amax, 1e-30f);
  const float r = __fdiv_rn(amax, 6.0f);
  float e = ceilf((float)log2((double)r));
  e = fminf(fmaxf(e, -127.0f), 127.0f);
  return (int)e;
}

// e2m1 code of y = x / 2^e: nearest of {0,.5,1,1.5,2,3,4,6}, ties to the smaller magnitude (the
// reference's first-index argmin), sign bit from (y < 0) whatever the magnitude.
UQ_DEV unsigned encode_e2m1(float x, float scale) {
  float y = __fdiv_rn(x, scale);
  y = fminf(fmaxf(y, -6.0f), 6.0f);
  const float a = fabsf(y);
  unsigned c = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
  return c | (y < 0.0f ? 8u : 0u);
}

template <typename T>
__global__ void __launch_bounds__(128) uq_append_kernel(uint8_t* __restrict__ kc, uint8_t* __restrict__ ks, uint8_t* __restrict__ vc,
                                                        uint8_t* __restrict__ vs, const T* __restrict__ key, const T* __restrict__ value,
                                                        const int64_t* __restrict__ slots, int T_tok, int HKV, int D, int PAGE, int nstream) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int total = T_tok * HKV * nstream;
  if (warp >= total) return;
  const int stream = warp % nstream;
  const int h = (warp / nstream) % HKV;
  const int t = warp / (nstream * HKV);
  const int64_t slot = slots[t];
  if (slot < 0) return;
  const int64_t page = slot / PAGE, off = slot % PAGE;
  const size_t row = ((size_t)page * HKV + h) * PAGE + off;
  const T* src = (stream == 0 ? key : value) + ((size_t)t * HKV + h) * D;
  uint8_t* codes = (stream == 0 ? kc : vc) + row * (D / 2);
  uint8_t* scales = (stream == 0 ? ks : vs) + row * (D / 32);
  for (int base = 0; base < D; base += 128) {
    const int ch = base + lane * 4;
    const bool live = ch < D;   // D = 64: lanes 16..31 idle
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
#pragma unroll
      for (int i = 0; i < 4; i++) x[i] = to_f32<T>(src[ch + i]);
    }
    float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
    for (int m = 1; m < 8; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    const int e = group_exponent(amax);
    // 2^e as fp32; e = -127 is the denormal 2^-127
    const float scale = e == -127 ? __int_as_float(0x00400000) : __int_as_float((e + 127) << 23);
    if (live) {
      const unsigned c0 = encode_e2m1(x[0], scale), c1 = encode_e2m1(x[1], scale);
      const unsigned c2 = encode_e2m1(x[2], scale), c3 = encode_e2m1(x[3], scale);
      *reinterpret_cast<uint16_t*>(codes + ch / 2) = (uint16_t)(c0 | (c1 << 4) | (c2 << 8) | (c3 << 12));
      if ((lane & 7) == 0) scales[ch / 32] = (uint8_t)(e + 127);
    }
  }
}

}  // namespace

// dtype: 0 fp32, 1 bf16, 2 fp16.  value/vc/vs may be null (single-stream form).
cudaError_t uq_append_dispatch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const void* key, const void* value,
                               const int64_t* slots, int T, int HKV, int D, int PAGE, int dtype, cudaStream_t s) {
  if (T == 0) return cudaSuccess;   // nothing to write; empty tensors may come with null pointers
  if (!kc || !ks || !key || !slots) return cudaErrorInvalidValue;
  const bool two = value != nullptr;
  if (two && (!vc || !vs)) return cudaErrorInvalidValue;
  if (!(D == 64 || D == 128 || D == 256) || PAGE <= 0 || HKV <= 0 || T < 0 || dtype < 0 || dtype > 2) return cudaErrorInvalidValue;
  const int nstream = two ? 2 : 1;
  const long long warps = (long long)T * HKV * nstream;
  const int blocks = (int)((warps + 3) / 4);
  switch (dtype) {
    case 0: uq_append_kernel<float><<<blocks, 128, 0, s>>>(kc, ks, vc, vs, (const float*)key, (const float*)value, slots, T, HKV, D, PAGE, nstream); break;
    case 1: uq_append_kernel<__nv_bfloat16><<<blocks, 128, 0, s>>>(kc, ks, vc, vs, (const __nv_bfloat16*)key, (const __nv_bfloat16*)value, slots, T, HKV, D, PAGE, nstream); break;
    default: uq_append_kernel<__half><<<blocks, 128, 0, s>>>(kc, ks, vc, vs, (const __half*)key, (const __half*)value, slots, T, HKV, D, PAGE, nstream); break;
  }
  return cudaGetLastError();
}
