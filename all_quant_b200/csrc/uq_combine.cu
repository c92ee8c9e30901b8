// Log-sum-exp combine of split-KV partials (the reference's uq_reduce_kernel, reference
// cuda/uq_decode.cu:353-388, restated): per query row,
//   mx = max_s lse_s;  w_s = 2^(lse_s - mx);  out = sum_s w_s * o_s / sum_s w_s;  all -inf -> zeros.
// One warp per output row; lanes stride the head dimension.  The same arithmetic serves: bf16 [B,K,Hq,D] (the op's
// result), fp32 partial + lse (one shard of a context split), that partial stored straight into every rank's exchange
// buffer over NVLink with a flag behind it (plain peer stores, no collective call), and the merge of R shards' partials
// into bf16, with or without a bounded wait for the R flags in front of it.
#include "uq_common.cuh"

namespace {

// Partials of (b, hk) live in scratch slots s = 0..ns_eff-1, rows r = j*G + g with stride BM.
// kOut: 0 bf16 result, 1 fp32 partial + lse2 to the caller's arrays, 2 the same partial to every rank's exchange buffer
template <int kOut>
__global__ void __launch_bounds__(128) uq_combine_kernel(const UQParams p, const UQLaunch x, float* __restrict__ o_part,
                                                         float* __restrict__ lse_part, const UQPeerPush push) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);   // over [B, K, HQ]
  const int lane = threadIdx.x & 31;
  const int total = p.B * p.K * p.HQ;
  // Launched as a programmatic dependent of the attention kernel (its blocks may become resident while that kernel's last
  // CTAs still run): nothing of the partials is read before the whole attention grid has completed and its writes are visible.
  // (A no-op when the launch carries no such dependency.)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (row < total) {
  const int h = row % p.HQ, j = (row / p.HQ) % p.K, b = row / (p.HQ * p.K);
  const int hk = h / x.G, r = j * x.G + (h % x.G);
  const int D = p.D;
  const size_t orow = uq_draft_row(x, b, j) * p.HQ + h;   // the row of the caller's [B, K, HQ] arrays (a chunk of drafts writes its own rows)
  const size_t slot0 = uq_slot(p, b, hk, 0);
  // The slots' log-sum-exps are read lane-parallel (slot s by lane s mod 32: up to four per lane for nsplit <= 128), so the
  // row's maximum, weights and denominator cost a few loads instead of a serial chain of nsplit of them.
  const int ns = x.ns_eff;
  float lse[4], w[4];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int s = lane + 32 * j;
    lse[j] = s < ns ? p.ml[(slot0 + s) * x.BM + r] : -INFINITY;
    mx = fmaxf(mx, lse[j]);
  }
#pragma unroll
  for (int m = 16; m; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
  float acc[8];   // D <= 256: 8 channels per lane
#pragma unroll
  for (int i = 0; i < 8; i++) acc[i] = 0.f;
  float den = 0.f;
  if (mx != -INFINITY) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      w[j] = lse[j] == -INFINITY ? 0.f : exp2f(lse[j] - mx);   // an empty split never wrote its o
      den += w[j];
    }
#pragma unroll
    for (int m = 16; m; m >>= 1) den += __shfl_xor_sync(0xffffffffu, den, m);
    for (int j = 0; j < 4 && 32 * j < ns; j++) {
      const unsigned live = __ballot_sync(0xffffffffu, w[j] != 0.f);
      for (unsigned rest = live; rest;) {
        // up to four non-empty slots at a time: their loads are in flight together
        int sl[4];
        float ws[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          sl[u] = rest ? __ffs(rest) - 1 : -1;
          if (rest) rest &= rest - 1;
          ws[u] = __shfl_sync(0xffffffffu, w[j], sl[u] < 0 ? 0 : sl[u]);
        }
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const float* o = p.mo + ((slot0 + 32 * j + (sl[u] < 0 ? 0 : sl[u])) * x.BM + r) * (size_t)D;
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int d = lane + 32 * i;
            v[u][i] = (sl[u] >= 0 && d < D) ? o[d] : 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
          if (sl[u] < 0) continue;
#pragma unroll
          for (int i = 0; i < 8; i++) acc[i] = fmaf(ws[u], v[u][i], acc[i]);
        }
      }
    }
  }
  // A wait of the attention kernel that ran out (status code set, not yet read by the host) leaves partials unwritten: the rows
  // are then NaN rather than numbers that look like an answer, so that a caller sees the failure without a synchronising read
  // of the status record.
  const float inv = x.status[0] != 0u ? __int_as_float(0x7fc00000) : (den > 0.f ? 1.f / den : 0.f) * x.out_scale;
  if (kOut == 1) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int d = lane + 32 * i;
      if (d < D) o_part[orow * D + d] = acc[i] * inv;
    }
    if (lane == 0) lse_part[orow] = den > 0.f ? mx + log2f(den) : -INFINITY;
  } else if (kOut == 2) {
    const float lse2 = den > 0.f ? mx + log2f(den) : -INFINITY;
    for (int r = 0; r < push.world; r++) {   // plain stores into each rank's buffer (the local one included)
      float* dst = push.slot[r];
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int d = lane + 32 * i;
        if (d < D) dst[orow * D + d] = acc[i] * inv;
      }
      if (lane == 0) dst[push.rows_total * D + orow] = lse2;
    }
  } else {
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + orow * D;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int d = lane + 32 * i;
      if (d < D) out[d] = __float2bfloat16_rn(acc[i] * inv);
    }
  }
  }
  if (kOut == 2 && push.raise) {
    // the block that finishes last raises this rank's flag on every rank: each block's stores are fenced at system scope
    // before its ticket, and the last ticket holder fences again before the flags, so whoever sees a flag sees the partial
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int ticket = atomicAdd(push.counter, 1u);
      if (ticket == gridDim.x - 1) {
        __threadfence_system();
        for (int r = 0; r < push.world; r++) *reinterpret_cast<volatile unsigned int*>(push.flag[r]) = push.seq;
        *push.counter = 0u;
      }
    }
  }
}

UQ_DEV unsigned int load_acquire_sys(const unsigned int* ptr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
UQ_DEV unsigned long long timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Merge of R shards: o [R, rows, D], lse2 [R, rows] -> bf16 [rows, D].  The shards may be apart by any stride (in floats):
// rows * D and rows for two plain arrays, rows * (D + 1) for both when every shard is one packed buffer (o, then lse2).
// flags != nullptr: thread r of every block first waits until flags[r] == seq (rank r's partial has arrived in this rank's
// exchange buffer), for wait_ns nanoseconds at most; when a wait runs out the status record gets code 3 with the rank and
// the sequence number, nothing is written and the kernel returns.
__global__ void __launch_bounds__(128) uq_merge_kernel(const float* o, const float* lse, int R, size_t rows, int D,
                                                       size_t o_stride, size_t l_stride, __nv_bfloat16* __restrict__ out,
                                                       const unsigned int* flags, unsigned int seq, unsigned long long wait_ns, unsigned int* status) {
  if (flags) {
    int arrived = 1;
    if ((int)threadIdx.x < R) {
      const unsigned long long t0 = timer_ns();
      while (load_acquire_sys(flags + threadIdx.x) != seq) {
        if (timer_ns() - t0 > wait_ns) { arrived = 0; break; }
        __nanosleep(40);
      }
      if (!arrived) uq_report(status, 3u, threadIdx.x, seq);
    }
    if (!__syncthreads_and(arrived)) return;
  }
  const size_t row = (size_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float mx = -INFINITY;
  for (int r = 0; r < R; r++) mx = fmaxf(mx, lse[(size_t)r * l_stride + row]);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; i++) acc[i] = 0.f;
  float den = 0.f;
  if (mx != -INFINITY) {
    for (int r = 0; r < R; r++) {
      const float l = lse[(size_t)r * l_stride + row];
      if (l == -INFINITY) continue;
      const float w = exp2f(l - mx);
      den += w;
      const float* src = o + (size_t)r * o_stride + row * D;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(w, src[d], acc[i]);
      }
    }
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int d = lane + 32 * i;
    if (d < D) out[row * D + d] = __float2bfloat16_rn(acc[i] * inv);
  }
}

}  // namespace

cudaError_t uq_combine_dispatch(const UQParams& p, const UQLaunch& x, float* o_part, float* lse_part, const UQPeerPush* push, bool pdl, cudaStream_t s) {
  const int rows = p.B * p.K * p.HQ;
  if (rows == 0) return cudaSuccess;
  const UQPeerPush none{};
  // programmatic stream serialisation: the launch may be set up while the attention kernel before it on the stream is still
  // running (that kernel signals early); the combine's first instruction waits for that kernel's completion
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((rows + 3) / 4);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  float* no_f = nullptr;
  if (push) return cudaLaunchKernelEx(&cfg, uq_combine_kernel<2>, p, x, no_f, no_f, *push);
  if (o_part) return cudaLaunchKernelEx(&cfg, uq_combine_kernel<1>, p, x, o_part, lse_part, none);
  return cudaLaunchKernelEx(&cfg, uq_combine_kernel<0>, p, x, no_f, no_f, none);
}

cudaError_t uq_merge_dispatch(const float* o, const float* lse, int R, size_t rows, int D, void* out, cudaStream_t s) {
  if (!o || !lse || !out || R < 1 || D < 32 || D > 256 || D % 32) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  uq_merge_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, s>>>(o, lse, R, rows, D, rows * D, rows, reinterpret_cast<__nv_bfloat16*>(out), nullptr, 0u, 0ull, nullptr);
  return cudaGetLastError();
}

// packed [R][rows * D + rows]: shard r's partial outputs, then its lse2 values (what one all-gather of per-rank buffers gives)
cudaError_t uq_merge_packed_dispatch(const float* packed, int R, size_t rows, int D, void* out, cudaStream_t s) {
  if (!packed || !out || R < 1 || D < 32 || D > 256 || D % 32) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  const size_t stride = rows * D + rows;
  uq_merge_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, s>>>(packed, packed + rows * D, R, rows, D, stride, stride, reinterpret_cast<__nv_bfloat16*>(out), nullptr, 0u, 0ull, nullptr);
  return cudaGetLastError();
}

// The merge of a context split over peer memory: the R slots of this rank's exchange buffer (parity seq & 1), each rank's
// partial awaited through its flag.  `own` is the buffer's base, slot_floats its slot size.
cudaError_t uq_merge_wait_dispatch(const void* own, int R, size_t slot_floats, unsigned int seq, size_t rows, int D, void* out,
                                   unsigned long long wait_ns, unsigned int* status, cudaStream_t s) {
  if (!own || !out || !status || R < 1 || R > kMaxPeers || D < 32 || D > 256 || D % 32 || rows * (size_t)(D + 1) > slot_floats) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  const int parity = (int)(seq & 1u);
  const float* data = reinterpret_cast<const float*>(own) + (size_t)parity * R * slot_floats;
  const unsigned int* flags = reinterpret_cast<const unsigned int*>(reinterpret_cast<const char*>(own) + uq_peer_data_bytes(R, slot_floats)) + parity * kMaxPeers;
  uq_merge_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, s>>>(data, data + rows * D, R, rows, D, slot_floats, slot_floats, reinterpret_cast<__nv_bfloat16*>(out), flags, seq, wait_ns, status);
  return cudaGetLastError();
}
