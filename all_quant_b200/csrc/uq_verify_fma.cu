// Verify/decode attention over the paged FP4 cache on the CUDA cores: the path for few query rows
// (K * group small) and the general path for every shape the tensor-core kernel does not take
// (head_dim 64/128/256, any page size).  Same operation as the reference's split kernels
// (reference cuda/uq_decode.cu:114-350) and CPU oracle (reference uqmt/attn.py:402-422); the kernel
// design is this library's own.
//
// Grid (split, kv head, sequence), 128 threads.  A CTA walks its page range in tiles of 128 keys and
// handles the query rows in chunks of RC, all rows of a chunk sharing each key that is read:
//   phase 1  thread = key:   load the key's D/2 code bytes and D/32 scale bytes straight from HBM
//                            (one row of the cache is contiguous), decode in registers, dot with the
//                            RC query rows held in shared memory, mask by the row's causal limit.
//   phase 2  warp = row:     running max / sum in the exp2 domain, scores -> probabilities in place.
//   phase 3  thread = channel pair: P.V with the value bytes read coalesced, decoded in registers.
// Each (sequence, kv head, split) writes a normalised partial (o, m + log2 l) to the caller's scratch.
//
// FMT 0 is the UltraQuant cache (one UE8M0 scale byte per 32 channels).  FMT 1 is the NVFP4 cache (reference
// uqmt/nvfp4.py:257-278, cuda/uq_decode.cu:604,384): one e4m3fn scale byte per 16 channels; the per-tensor scales
// are not applied here: k_ts rides in the softmax scale and v_ts multiplies the combined output.
#include "uq_common.cuh"

namespace {

constexpr int kTile = 128;   // keys per tile = threads per CTA

template <int D, int RC, int FMT>
__global__ void __launch_bounds__(kTile) uq_verify_fma_kernel(const UQParams p, const UQLaunch x) {
  constexpr int NG = D / 32;            // 16-byte code groups per row
  constexpr int NS = FMT ? D / 16 : D / 32;   // scale bytes per row
  constexpr int KPAR = 256 / D < 1 ? 1 : 256 / D;   // key phases in P.V: threads / (D/2) = 128 / (D/2)
  const int s = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  __shared__ __align__(16) float q_s[RC][D];
  __shared__ __align__(16) float p_s[RC][kTile];
  __shared__ unsigned long long row_s[kTile];
  __shared__ float m_s[RC], l_s[RC], a_s[RC];
  __shared__ float red_s[KPAR > 1 ? (KPAR - 1) * RC * D : 1];

  int off;
  const int n_loc = uq_n_local(p, x, b, &off);
  const int n_glob = uq_seq_len(p, x, b);
  const int n_pages = (n_loc + p.PAGE - 1) / p.PAGE;
  const int pps = (n_pages + x.ns_eff - 1) / x.ns_eff;
  const int k0 = min(s * pps, n_pages) * p.PAGE;
  const int k1 = min(min((s + 1) * pps, n_pages) * p.PAGE, n_loc);
  const size_t slot = uq_slot(p, b, hk, s);
  float* mo = p.mo + slot * x.BM * D;
  float* ml = p.ml + slot * x.BM;
  const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(p.q);

  for (int r0 = 0; r0 < x.rows; r0 += RC) {
    // stage the chunk's query rows as fp32
    for (int i = tid; i < RC * D; i += kTile) {
      const int r = r0 + i / D, d = i % D;
      float v = 0.f;
      if (r < x.rows) {
        const int j = r / x.G, g = r % x.G;
        v = __bfloat162float(q[(uq_draft_row(x, b, j) * p.HQ + hk * x.G + g) * D + d]);
      }
      q_s[i / D][d] = v;
    }
    if (tid < RC) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
    float o[RC][2];
#pragma unroll
    for (int r = 0; r < RC; r++) o[r][0] = o[r][1] = 0.f;
    __syncthreads();

    for (int t0 = k0; t0 < k1; t0 += kTile) {
      // ---- phase 1: scores
      {
        const int key = t0 + tid;
        float acc[RC];
#pragma unroll
        for (int r = 0; r < RC; r++) acc[r] = 0.f;
        const bool live = key < k1;
        if (live) {
          const size_t row = ((size_t)p.block_table[(size_t)b * p.max_pages + key / p.PAGE] * p.HKV + hk) * p.PAGE + key % p.PAGE;
          row_s[tid] = row;
          const uint4* codes = reinterpret_cast<const uint4*>(p.kc + row * (D / 2));
          const uint8_t* sc = p.ks + row * NS;
#pragma unroll
          for (int g = 0; g < NG; g++) {
            const uint4 c4 = __ldg(codes + g);
            const float sc_lo = FMT ? uq_e4m3_f32(__ldg(sc + 2 * g)) : uq_scale_f32(__ldg(sc + g));
            const float sc_hi = FMT ? uq_e4m3_f32(__ldg(sc + 2 * g + 1)) : sc_lo;
            const unsigned w[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
            for (int wi = 0; wi < 4; wi++) {
              const float scale = wi < 2 ? sc_lo : sc_hi;
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; i++) f[i] = uq_e2m1_f32((w[wi] >> (4 * i)) & 0xFu) * scale;
#pragma unroll
              for (int r = 0; r < RC; r++) {
                const float4 qa = *reinterpret_cast<const float4*>(&q_s[r][g * 32 + wi * 8]);
                const float4 qb = *reinterpret_cast<const float4*>(&q_s[r][g * 32 + wi * 8 + 4]);
                acc[r] = fmaf(f[0], qa.x, acc[r]); acc[r] = fmaf(f[1], qa.y, acc[r]);
                acc[r] = fmaf(f[2], qa.z, acc[r]); acc[r] = fmaf(f[3], qa.w, acc[r]);
                acc[r] = fmaf(f[4], qb.x, acc[r]); acc[r] = fmaf(f[5], qb.y, acc[r]);
                acc[r] = fmaf(f[6], qb.z, acc[r]); acc[r] = fmaf(f[7], qb.w, acc[r]);
              }
            }
          }
        }
        const int pos = off + key;   // global position of this key
#pragma unroll
        for (int r = 0; r < RC; r++) {
          const int rr = r0 + r;
          // the committed prefix is visible to every row; a draft position to the rows whose query may attend it
          const int td = pos - (n_glob - p.K);
          const bool vis = live && rr < x.rows && pos < n_glob && (td < 0 || uq_sees_draft(p, x, b, rr / x.G, td));
          p_s[r][tid] = vis ? acc[r] * x.sc2 : -INFINITY;
        }
      }
      __syncthreads();
      // ---- phase 2: online softmax, one warp per row
      for (int r = warp; r < RC; r += kTile / 32) {
        float v[4], mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; i++) { v[i] = p_s[r][lane + 32 * i]; mx = fmaxf(mx, v[i]); }
#pragma unroll
        for (int m = 16; m; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
        const float m_old = m_s[r];
        const float m_new = fmaxf(m_old, mx);
        const float base = m_new == -INFINITY ? 0.f : m_new;   // all masked so far: exp2(-inf - 0) = 0
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) { const float pv = exp2f(v[i] - base); p_s[r][lane + 32 * i] = pv; sum += pv; }
#pragma unroll
        for (int m = 16; m; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
        if (lane == 0) {
          const float alpha = exp2f(m_old - base);   // m_old = -inf -> 0
          a_s[r] = alpha;
          m_s[r] = m_new;
          l_s[r] = l_s[r] * alpha + sum;
        }
      }
      __syncthreads();
      // ---- phase 3: o += P.V, thread = one byte (two channels) of the value row
      {
        const int dbyte = tid % (D / 2), kpar = tid / (D / 2);
#pragma unroll
        for (int r = 0; r < RC; r++) { const float al = a_s[r]; o[r][0] *= al; o[r][1] *= al; }
        const int kend = min(kTile, k1 - t0);
        for (int kk = kpar; kk < kend; kk += KPAR) {
          const size_t row = row_s[kk];
          const unsigned byte = __ldg(p.vc + row * (D / 2) + dbyte);
          const float scale = FMT ? uq_e4m3_f32(__ldg(p.vs + row * NS + dbyte / 8)) : uq_scale_f32(__ldg(p.vs + row * NS + dbyte / 16));
          const float v0 = uq_e2m1_f32(byte & 0xFu) * scale, v1 = uq_e2m1_f32(byte >> 4) * scale;
#pragma unroll
          for (int r = 0; r < RC; r++) {
            const float pv = p_s[r][kk];
            // a masked key has pv == 0 exactly; its value bytes may be anything (inf scale included)
            if (pv != 0.f) { o[r][0] = fmaf(pv, v0, o[r][0]); o[r][1] = fmaf(pv, v1, o[r][1]); }
          }
        }
      }
      __syncthreads();
    }

    // ---- write the partial of this row chunk
    {
      const int dbyte = tid % (D / 2), kpar = tid / (D / 2);
      if (KPAR > 1) {
        if (kpar > 0) {
#pragma unroll
          for (int r = 0; r < RC; r++) {
            red_s[((kpar - 1) * RC + r) * D + 2 * dbyte] = o[r][0];
            red_s[((kpar - 1) * RC + r) * D + 2 * dbyte + 1] = o[r][1];
          }
        }
        __syncthreads();
      }
      if (kpar == 0) {
#pragma unroll
        for (int r = 0; r < RC; r++) {
          const int rr = r0 + r;
          if (rr >= x.rows) continue;
          float a0 = o[r][0], a1 = o[r][1];
          for (int kp = 1; kp < KPAR; kp++) {
            a0 += red_s[((kp - 1) * RC + r) * D + 2 * dbyte];
            a1 += red_s[((kp - 1) * RC + r) * D + 2 * dbyte + 1];
          }
          const float l = l_s[r];
          const float inv = l > 0.f ? 1.f / l : 0.f;
          *reinterpret_cast<float2*>(mo + (size_t)rr * D + 2 * dbyte) = make_float2(a0 * inv, a1 * inv);
        }
      }
      if (tid < RC && r0 + tid < x.rows) {
        const float l = l_s[tid];
        ml[r0 + tid] = l > 0.f ? m_s[tid] + log2f(l) : -INFINITY;
      }
    }
    __syncthreads();
  }
}

template <int D, int FMT>
cudaError_t launch_f(const UQParams& p, const UQLaunch& x, cudaStream_t s) {
  const dim3 grid(x.ns_eff, p.HKV, p.B);
  if (x.rows <= 4)
    uq_verify_fma_kernel<D, 4, FMT><<<grid, kTile, 0, s>>>(p, x);
  else
    uq_verify_fma_kernel<D, 8, FMT><<<grid, kTile, 0, s>>>(p, x);
  return cudaGetLastError();
}

template <int D>
cudaError_t launch_d(const UQParams& p, const UQLaunch& x, cudaStream_t s) {
  return p.fmt == 1 ? launch_f<D, 1>(p, x, s) : launch_f<D, 0>(p, x, s);
}

}  // namespace

cudaError_t uq_verify_fma_dispatch(const UQParams& p, const UQLaunch& x, cudaStream_t s) {
  switch (p.D) {
    case 64: return launch_d<64>(p, x, s);
    case 128: return launch_d<128>(p, x, s);
    case 256: return launch_d<256>(p, x, s);
  }
  return cudaErrorInvalidValue;
}
