/* Argument block of the verify/decode attention launch.  Field order, types and size (136 bytes on
 * LP64) are those of the reference's `struct UQParams` (reference cuda/uq_decode.h:11-30); a caller
 * that fills the reference's struct can pass it here unchanged.  Plain C so that it can be mirrored
 * by ctypes / cgo / JNI without a C++ compiler. */
#ifndef UQ_PARAMS_H_
#define UQ_PARAMS_H_
#include <stdint.h>

typedef struct UQParams {
  const void* q;              /* bf16 [B,K,Hq,D] */
  const uint8_t* kc;          /* [pages,Hkv,PAGE,D/2] */
  const uint8_t* ks;          /* [pages,Hkv,PAGE,D/32] */
  const uint8_t* vc;
  const uint8_t* vs;
  const int32_t* block_table; /* [B,max_pages] */
  const int32_t* seq_lens;    /* [B], includes the K draft tokens */
  float* mo;                  /* scratch: fp32 [B,Hkv,nsplit,BLOCK_M,D] partial outputs */
  float* ml;                  /* scratch: fp32 [B,Hkv,nsplit,BLOCK_M]   partial log2-sum-exp */
  void* out;                  /* bf16 [B,K,Hq,D] */
  int B, K, HQ, HKV, D, PAGE, max_pages;
  int nsplit;                 /* partial slots per (sequence, kv head) in the scratch: 1..128 */
  float sm_scale;
  int variant;                /* kernel selector of the reference (0..4): accepted, ignored */
  int mb;                     /* tuning hint of the reference: accepted, ignored */
  int fmt;                    /* 0 = UE8M0 scale per 32 channels; 1 = NVFP4: e4m3fn scale per 16 channels (ks/vs [.., D/16]) */
  float k_ts, v_ts;           /* fmt 1 only: k_ts scales the scores, v_ts the output (1.0 = none) */
} UQParams;

#endif
