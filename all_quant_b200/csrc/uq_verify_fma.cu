// Verify/decode attention over the paged FP4 cache on the CUDA cores: the path for few query rows
// (K * group small) and the general path for every shape the tensor-core kernel does not take
// (head_dim 64/128/256, any page size).  Same operation as the reference's split kernels
// (reference cuda/uq_decode.cu:114-350) and CPU oracle (reference uqmt/attn.py:402-422); the kernel
// design is this library's own.
//
// Grid (split, kv head, sequence), 128 threads.  A CTA walks its page range in tiles of 128 keys; a tile's K and V rows
// (codes and scale bytes) are copied to shared memory once and serve all query rows of a pass (up to 32, in chunks of RC):
//   stage    thread = key:   the key's code rows and scale bytes of K and V, cache -> shared memory (a row is contiguous).
//   phase 1  thread = key:   decode the staged K row in registers, dot with the chunk's RC query rows (fp32 in shared
//                            memory), mask by the row's causal limit (or its tree mask).
//   phase 2  warp = row:     running max / sum in the exp2 domain, scores -> probabilities in place.
//   phase 3  thread = channel pair: P.V from the staged value rows, decoded in registers.
// Each (sequence, kv head, split) writes a normalised partial (o, m + log2 l) to the caller's scratch.
//
// FMT 0 is the UltraQuant cache (one UE8M0 scale byte per 32 channels).  FMT 1 is the NVFP4 cache (reference
// uqmt/nvfp4.py:257-278, cuda/uq_decode.cu:604,384): one e4m3fn scale byte per 16 channels; the per-tensor scales
// are not applied here: k_ts rides in the softmax scale and v_ts multiplies the combined output.
#include <atomic>

#include "uq_common.cuh"

namespace {

constexpr int kTile = 128;   // keys per tile = threads per CTA

// bytes of one staged cache row (codes, then scale bytes), padded so that the rows of a quarter warp fall on different banks
__host__ __device__ constexpr int row_stride(int D, int FMT) {
  const int raw = D / 2 + (FMT ? D / 16 : D / 32);
  const int r16 = (raw + 15) / 16;
  return (r16 % 2 ? r16 : r16 + 1) * 16;
}
template <int D, int RC, int NCH, int FMT>
struct Smem {
  static constexpr int kStride = row_stride(D, FMT);
  static constexpr int oK = 0, oV = oK + kTile * kStride, oQ = oV + kTile * kStride;   // K rows, V rows, then fp32 [RC * NCH][D] queries
  static constexpr int oP = oQ + RC * NCH * D * 4;                                       // fp32 [RC][kTile] scores / probabilities of the chunk
  static constexpr int oM = oP + RC * kTile * 4;                                         // fp32 [RC * NCH] running maxima, then sums, then [RC] factors
  static constexpr int kBytes = oM + (2 * RC * NCH + RC) * 4;
};

// One pass = RC * NCH query rows (at most 32).  Every 128-key tile of the CTA's page range is copied from the cache to shared
// memory ONCE per pass (thread = key: its code row and scale bytes of K and of V) and all row chunks of the pass are served
// from that copy: the row loop sits inside the key loop, so K = 8 with a group of 4 reads the cache once, not once per chunk.
template <int D, int RC, int NCH, int FMT>
__global__ void __launch_bounds__(kTile) uq_verify_fma_kernel(const UQParams p, const UQLaunch x) {
  using S = Smem<D, RC, NCH, FMT>;
  constexpr int NG = D / 32;                  // 16-byte code groups per row
  constexpr int NS = FMT ? D / 16 : D / 32;   // scale bytes per row
  constexpr int KPAR = 256 / D < 1 ? 1 : 256 / D;   // key phases in P.V: threads / (D/2) = 128 / (D/2)
  constexpr int RS = RC * NCH;
  const int s = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  extern __shared__ __align__(16) uint8_t sm[];
  uint8_t* k_s = sm + S::oK;
  uint8_t* v_s = sm + S::oV;
  float (*q_s)[D] = reinterpret_cast<float (*)[D]>(sm + S::oQ);
  float (*p_s)[kTile] = reinterpret_cast<float (*)[kTile]>(sm + S::oP);
  float* m_s = reinterpret_cast<float*>(sm + S::oM);
  float* l_s = m_s + RS;
  float* a_s = l_s + RS;

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
  const int dbyte = tid % (D / 2), kpar = tid / (D / 2);   // P.V: this thread's byte (two channels) of the value row and its key phase

  for (int r0 = 0; r0 < x.rows; r0 += RS) {
    // the pass's query rows as fp32
    for (int i = tid; i < RS * D; i += kTile) {
      const int r = r0 + i / D, d = i % D;
      float v = 0.f;
      if (r < x.rows) {
        const int j = r / x.G, g = r % x.G;
        v = __bfloat162float(q[(uq_draft_row(x, b, j) * p.HQ + hk * x.G + g) * D + d]);
      }
      q_s[i / D][d] = v;
    }
    if (tid < RS) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
    float o[NCH][RC][2];
#pragma unroll
    for (int c = 0; c < NCH; c++)
#pragma unroll
      for (int r = 0; r < RC; r++) o[c][r][0] = o[c][r][1] = 0.f;
    __syncthreads();

    for (int t0 = k0; t0 < k1; t0 += kTile) {
      // ---- the tile's rows: cache -> shared memory, once
      const int key = t0 + tid;
      const bool live = key < k1;
      if (live) {
        const size_t row = ((size_t)p.block_table[(size_t)b * p.max_pages + key / p.PAGE] * p.HKV + hk) * p.PAGE + key % p.PAGE;
        const uint4* kc4 = reinterpret_cast<const uint4*>(p.kc + row * (D / 2));   // (kc is 16-byte aligned: the launch checks it)
        uint4* kd = reinterpret_cast<uint4*>(k_s + tid * S::kStride);
#pragma unroll
        for (int g = 0; g < NG; g++) kd[g] = __ldg(kc4 + g);
        const uint8_t* vc1 = p.vc + row * (D / 2);                                // (vc, ks, vs may have any alignment)
        uint8_t* vd = v_s + tid * S::kStride;
        if ((reinterpret_cast<uintptr_t>(vc1) & 15) == 0) {
#pragma unroll
          for (int g = 0; g < NG; g++) reinterpret_cast<uint4*>(vd)[g] = __ldg(reinterpret_cast<const uint4*>(vc1) + g);
        } else {
          for (int i = 0; i < D / 2; i++) vd[i] = __ldg(vc1 + i);
        }
#pragma unroll
        for (int i = 0; i < NS; i++) {
          k_s[tid * S::kStride + D / 2 + i] = __ldg(p.ks + row * NS + i);
          vd[D / 2 + i] = __ldg(p.vs + row * NS + i);
        }
      }
      __syncthreads();
      const int pos = off + key;   // global position of this thread's key
      const int td = pos - (n_glob - p.K);
#pragma unroll
      for (int c = 0; c < NCH; c++) {
        if (r0 + c * RC >= x.rows) break;
        // ---- phase 1: scores of the chunk's rows, thread = key
        {
          float acc[RC];
#pragma unroll
          for (int r = 0; r < RC; r++) acc[r] = 0.f;
          if (live) {
            const uint4* codes = reinterpret_cast<const uint4*>(k_s + tid * S::kStride);
            const uint8_t* sc = k_s + tid * S::kStride + D / 2;
#pragma unroll
            for (int g = 0; g < NG; g++) {
              const uint4 c4 = codes[g];
              const float sc_lo = FMT ? uq_e4m3_f32(sc[2 * g]) : uq_scale_f32(sc[g]);
              const float sc_hi = FMT ? uq_e4m3_f32(sc[2 * g + 1]) : sc_lo;
              const unsigned w[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
              for (int wi = 0; wi < 4; wi++) {
                const float scale = wi < 2 ? sc_lo : sc_hi;
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; i++) f[i] = uq_e2m1_f32((w[wi] >> (4 * i)) & 0xFu) * scale;
#pragma unroll
                for (int r = 0; r < RC; r++) {
                  const float4 qa = *reinterpret_cast<const float4*>(&q_s[c * RC + r][g * 32 + wi * 8]);
                  const float4 qb = *reinterpret_cast<const float4*>(&q_s[c * RC + r][g * 32 + wi * 8 + 4]);
                  acc[r] = fmaf(f[0], qa.x, acc[r]); acc[r] = fmaf(f[1], qa.y, acc[r]);
                  acc[r] = fmaf(f[2], qa.z, acc[r]); acc[r] = fmaf(f[3], qa.w, acc[r]);
                  acc[r] = fmaf(f[4], qb.x, acc[r]); acc[r] = fmaf(f[5], qb.y, acc[r]);
                  acc[r] = fmaf(f[6], qb.z, acc[r]); acc[r] = fmaf(f[7], qb.w, acc[r]);
                }
              }
            }
          }
#pragma unroll
          for (int r = 0; r < RC; r++) {
            const int rr = r0 + c * RC + r;
            // the committed prefix is visible to every row; a draft position to the rows whose query may attend it
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
          const float m_old = m_s[c * RC + r];
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
            m_s[c * RC + r] = m_new;
            l_s[c * RC + r] = l_s[c * RC + r] * alpha + sum;
          }
        }
        __syncthreads();
        // ---- phase 3: o += P.V from the staged value rows, thread = one byte (two channels)
        {
#pragma unroll
          for (int r = 0; r < RC; r++) { const float al = a_s[r]; o[c][r][0] *= al; o[c][r][1] *= al; }
          const int kend = min(kTile, k1 - t0);
          for (int kk = kpar; kk < kend; kk += KPAR) {
            const uint8_t* vrow = v_s + kk * S::kStride;
            const unsigned byte = vrow[dbyte];
            const float scale = FMT ? uq_e4m3_f32(vrow[D / 2 + dbyte / 8]) : uq_scale_f32(vrow[D / 2 + dbyte / 16]);
            const float v0 = uq_e2m1_f32(byte & 0xFu) * scale, v1 = uq_e2m1_f32(byte >> 4) * scale;
#pragma unroll
            for (int r = 0; r < RC; r++) {
              const float pv = p_s[r][kk];
              // a masked key has pv == 0 exactly; its value bytes may be anything (inf scale included)
              if (pv != 0.f) { o[c][r][0] = fmaf(pv, v0, o[c][r][0]); o[c][r][1] = fmaf(pv, v1, o[c][r][1]); }
            }
          }
        }
        __syncthreads();
      }
    }

    // ---- write the partials of this pass (the key phases of a channel pair are added through shared memory: the staged K rows
    // are free by now)
    float* red_s = reinterpret_cast<float*>(sm + S::oK);   // [KPAR - 1][RC][D]
    static_assert((KPAR > 1 ? (KPAR - 1) * RC * D * 4 : 0) <= 2 * kTile * Smem<D, RC, NCH, FMT>::kStride, "reduction scratch fits the staged rows");
#pragma unroll
    for (int c = 0; c < NCH; c++) {
      if (r0 + c * RC >= x.rows) break;
      if (KPAR > 1) {
        if (kpar > 0) {
#pragma unroll
          for (int r = 0; r < RC; r++) {
            red_s[((kpar - 1) * RC + r) * D + 2 * dbyte] = o[c][r][0];
            red_s[((kpar - 1) * RC + r) * D + 2 * dbyte + 1] = o[c][r][1];
          }
        }
        __syncthreads();
      }
      if (kpar == 0) {
#pragma unroll
        for (int r = 0; r < RC; r++) {
          const int rr = r0 + c * RC + r;
          if (rr >= x.rows) continue;
          float a0 = o[c][r][0], a1 = o[c][r][1];
          for (int kp = 1; kp < KPAR; kp++) {
            a0 += red_s[((kp - 1) * RC + r) * D + 2 * dbyte];
            a1 += red_s[((kp - 1) * RC + r) * D + 2 * dbyte + 1];
          }
          const float l = l_s[c * RC + r];
          const float inv = l > 0.f ? 1.f / l : 0.f;
          *reinterpret_cast<float2*>(mo + (size_t)rr * D + 2 * dbyte) = make_float2(a0 * inv, a1 * inv);
        }
      }
      if (KPAR > 1) __syncthreads();
    }
    if (tid < RS && r0 + tid < x.rows) {
      const float l = l_s[tid];
      ml[r0 + tid] = l > 0.f ? m_s[tid] + log2f(l) : -INFINITY;
    }
    __syncthreads();
  }
}

template <int D, int RC, int NCH, int FMT>
cudaError_t launch_k(const UQParams& p, const UQLaunch& x, cudaStream_t s) {
  using S = Smem<D, RC, NCH, FMT>;
  auto kern = uq_verify_fma_kernel<D, RC, NCH, FMT>;
  static std::atomic<bool> ready[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (S::kBytes > 48 * 1024 && !ready[dev].load(std::memory_order_acquire)) {   // per device: more than the default dynamic shared memory
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
    if (e != cudaSuccess) { cudaGetLastError(); return e; }
    ready[dev].store(true, std::memory_order_release);
  }
  kern<<<dim3(x.ns_eff, p.HKV, p.B), kTile, S::kBytes, s>>>(p, x);
  return cudaGetLastError();
}

template <int D, int FMT>
cudaError_t launch_f(const UQParams& p, const UQLaunch& x, cudaStream_t s) {
  // rows per pass: 4, 8, 16 or 32 (more rows: passes of 32, each reading the cache once)
  if (x.rows <= 4) return launch_k<D, 4, 1, FMT>(p, x, s);
  if (x.rows <= 8) return launch_k<D, 8, 1, FMT>(p, x, s);
  if (x.rows <= 16) return launch_k<D, 8, 2, FMT>(p, x, s);
  return launch_k<D, 8, 4, FMT>(p, x, s);
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
