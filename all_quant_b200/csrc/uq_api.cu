// Host side of libuq_b200: argument checks, kernel choice, and the exported entry points — the
// reference's C++ surface (include/uq_decode.h) and the C ABI (include/uq_b200.h).
//
// Dispatch (the reference's is a template tree over variant / BLOCK_M / warps / stages, reference
// cuda/uq_decode.cu:402-626; this library has two kernels and ignores those hints):
//   tcgen05 kernel  when head_dim, page size, alignment and row count are ones it serves (uq_verify_tc.cu): every
//                   page size that is a multiple of 16 from 16 to 1024 tokens, up to 64 rows per launch, 65-128 rows as draft chunks
//   CUDA-core kernel for everything else (uq_verify_fma.cu)
// followed by the combine kernel.  Every check happens before the first launch, so
// cudaErrorInvalidValue means nothing was enqueued (callers of the reference skip on it).
//
// Alignment contract (checked here; a pointer that breaks it is refused, never dereferenced): q and kc 16 bytes (both
// kernels read them as 16-byte vectors), mo 8 bytes, ml and out 4 bytes, the page table and seq_lens 4 bytes.  vc, ks and
// vs may have any alignment on the CUDA-core kernel; the tcgen05 kernel wants kc / vc / ks / vs 16-byte aligned (kc 32
// for the block-scaled head_dim 128) and a call that is not falls to the CUDA-core kernel.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "uq_b200.h"
#include "uq_common.cuh"
#include "uq_decode.h"

__device__ unsigned int g_uq_status[4];

// Built-in scratch of uqb_decode_launch_static: 24 MiB of fp32 partials, resident on every device that loads the
// library from the moment the module is loaded until the process exits.  In host code this name is only a handle
// for the runtime, never an address a kernel can use: the device address comes from cudaGetSymbolAddress.
constexpr size_t kStaticScratchFloats = (size_t)24 * 1024 * 1024 / sizeof(float);
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

cudaError_t uq_append_dispatch(uint8_t*, uint8_t*, uint8_t*, uint8_t*, const void*, const void*, const int64_t*, int, int, int, int, int, cudaStream_t, int flags, float c);
cudaError_t uq_fwht_dispatch(const void*, void*, long long, int, int, cudaStream_t);
cudaError_t uq_append_nvfp4_dispatch(uint8_t*, uint8_t*, uint8_t*, uint8_t*, const void*, const void*, const int64_t*, int, int, int, int, int, float, float, cudaStream_t, int route);
cudaError_t uq_verify_fma_dispatch(const UQParams&, const UQLaunch&, cudaStream_t);
cudaError_t uq_verify_tc_dispatch(const UQParams&, const UQLaunch&, cudaStream_t);
bool uq_verify_tc_serves(const UQParams&, const UQLaunch&);
int uq_verify_tc_splits(const UQParams&, const UQLaunch&);
cudaError_t uq_combine_dispatch(const UQParams&, const UQLaunch&, float*, float*, const UQPeerPush*, bool, cudaStream_t);
cudaError_t uq_merge_wait_dispatch(const void*, int, size_t, unsigned int, size_t, int, void*, unsigned long long, unsigned int*, cudaStream_t);
cudaError_t uq_merge_dispatch(const float*, const float*, int, size_t, int, void*, cudaStream_t);
cudaError_t uq_layout_dispatch(int, uint8_t*, uint8_t*, uint8_t*, uint8_t*, uint8_t*, long long, int, int, int, int, int, cudaStream_t);
cudaError_t uq_merge_packed_dispatch(const float*, int, size_t, int, void*, cudaStream_t);

namespace {

constexpr int kMaxDevices = 64;   // per-device tables (status record, attributes, scratch address); a device index beyond is refused
std::atomic<unsigned long long> g_launches{0};
thread_local int t_last_path = 0;
thread_local cudaEvent_t t_ev_before = nullptr, t_ev_after = nullptr;

int pow2ceil(int v) {   // saturates at 2^30 (an int cannot hold the next power)
  int p = 1;
  while (p < v && p < (1 << 30)) p <<= 1;
  return p;
}

// Argument ranges within which the size arithmetic below cannot overflow and the kernels' 32-bit indices hold.
bool sizes_ok(const UQParams& p) {
  if (p.B < 0 || p.B > (1 << 20) || p.K < 1 || p.K > 128 || p.HQ < 1 || p.HQ > (1 << 16) || p.HKV < 1 || p.HKV > p.HQ || p.HQ % p.HKV) return false;
  if (p.HQ / p.HKV > 128) return false;
  if (!(p.D == 64 || p.D == 128 || p.D == 256)) return false;
  return p.nsplit >= 1 && p.nsplit <= 128;
}

bool aligned(const void* ptr, uintptr_t a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) == 0; }

// UQ_B200_CFG="expire=30" makes the tcgen05 kernel's softmax role withhold one arrival (the query tile of a segment is never
// announced), so that the issuing thread's bounded wait on barrier 30 runs out after its second and the kernel's give-up path
// (status record, drain of the copies in flight, common exit) runs on a healthy GPU.  Tests only.
int forced_expire() {
  const char* e = std::getenv("UQ_B200_CFG");
  const char* at = e ? std::strstr(e, "expire=") : nullptr;
  return at ? std::atoi(at + 7) : 0;
}

// UQ_B200_CFG="path=fma" or "path=tc" forces a kernel (a forced tc on an unserved shape is invalid value).
int forced_path() {
  const char* e = std::getenv("UQ_B200_CFG");
  if (!e) return 0;
  if (std::strstr(e, "path=fma")) return 1;
  if (std::strstr(e, "path=tc")) return 2;
  return 0;
}

// Device address of the current device's status record (the symbol's name is only a host-side handle).
// (nullptr for a device index outside the per-device tables: the caller answers cudaErrorInvalidDevice)
unsigned int* status_ptr() {
  static std::atomic<unsigned int*> cached[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return nullptr; }
  unsigned int* ptr = cached[dev].load(std::memory_order_acquire);
  if (!ptr) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_uq_status) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    ptr = reinterpret_cast<unsigned int*>(sym);
    cached[dev].store(ptr, std::memory_order_release);   // (two threads racing here store the same address)
  }
  return ptr;
}

int sm_count() {
  static std::atomic<int> cached[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return 148; }
  int n = cached[dev].load(std::memory_order_relaxed);
  if (!n) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n > 0 ? n : 148;
}

bool shape_ok(const UQParams& p) {
  if (p.fmt != 0 && p.fmt != 1) return false;   // 0 UltraQuant, 1 NVFP4; both kernels serve both
  if (!sizes_ok(p)) return false;
  if (p.PAGE < 1 || p.max_pages < 0) return false;
  if (uq_block_m(p.K, p.HQ, p.HKV) > 128) return false;   // the reference's limit on rows per tile
  if (!(p.q && p.kc && p.ks && p.vc && p.vs && p.block_table && p.seq_lens && p.mo && p.ml)) return false;
  // the alignment contract (see the head of this file): refused here, before anything is enqueued
  if (!aligned(p.q, 16) || !aligned(p.kc, 16) || !aligned(p.mo, 8) || !aligned(p.ml, 4) || !aligned(p.block_table, 4) || !aligned(p.seq_lens, 4)) return false;
  return !p.out || aligned(p.out, 4);
}

cudaError_t run_one(const UQParams& p, UQLaunch x, float* o_part, float* lse_part, cudaStream_t s, const UQPeerPush* push);

cudaError_t run(const UQParams& p, const int32_t* pos_offset, float* o_part, float* lse_part, cudaStream_t s, const int32_t* tree_mask = nullptr,
                const UQPeerPush* push = nullptr) {
  if (!shape_ok(p)) return cudaErrorInvalidValue;
  if (tree_mask && p.K > 16) return cudaErrorInvalidValue;   // the reference's limit (uqmt/tree.py:135)
  if (!o_part && !p.out && !push) return cudaErrorInvalidValue;
  if (p.B == 0) return cudaSuccess;
  UQLaunch x{};
  x.pos_offset = pos_offset;
  x.tree_mask = tree_mask;
  x.k_first = 0;
  x.k_total = p.K;
  x.len_cut = 0;
  x.expire_id = forced_expire();
  x.status = status_ptr();
  if (!x.status) {
    int dev = -1;
    cudaGetDevice(&dev);
    return dev < 0 || dev >= kMaxDevices ? cudaErrorInvalidDevice : cudaErrorInitializationError;
  }
  // More query rows than the tensor-core kernel takes in one launch (K * group > 64, up to the 128 of uq_block_m): the
  // drafts are run as chunks of consecutive drafts, each a verify call of its own on the sequence cut after the chunk
  // (see UQLaunch), sharing the caller's scratch one after the other.  A tree-masked call is chunked without the cut: its
  // masks decide which of the caller's drafts a query sees, whichever chunk they belong to.
  const int G = p.HQ / p.HKV;
  const int per = G <= 64 ? 64 / G : 0;   // drafts per chunk
  if (p.K * G > 64 && per >= 1 && forced_path() != 1) {
    UQParams pc = p;
    pc.K = per;
    UQLaunch xc = x;
    xc.G = G;
    xc.rows = per * G;
    if (uq_verify_tc_serves(pc, xc)) {
      for (int k0 = 0; k0 < p.K; k0 += per) {
        pc.K = std::min(per, p.K - k0);
        xc.k_first = k0;
        xc.len_cut = tree_mask ? 0 : p.K - k0 - pc.K;
        UQPeerPush pp{};
        if (push) {   // every chunk stores its rows into the peers' buffers; the last one raises the flags
          pp = *push;
          pp.raise = k0 + per >= p.K;
        }
        cudaError_t e = run_one(pc, xc, o_part, lse_part, s, push ? &pp : nullptr);
        if (e != cudaSuccess) return e;
      }
      return cudaSuccess;
    }
  }
  return run_one(p, x, o_part, lse_part, s, push);
}

// One launch of a verify kernel and its combine; x carries the caller's pointers and the draft chunk.
cudaError_t run_one(const UQParams& p, UQLaunch x, float* o_part, float* lse_part, cudaStream_t s, const UQPeerPush* push) {
  x.G = p.HQ / p.HKV;
  x.rows = p.K * x.G;
  x.BM = uq_block_m(p.K, p.HQ, p.HKV);
  // NVFP4 (reference cuda/uq_decode.cu:604,384): k_ts is folded into the softmax scale, v_ts multiplies the output
  x.sc2 = p.sm_scale * (p.fmt == 1 ? p.k_ts : 1.f) * 1.4426950408889634f;
  x.out_scale = p.fmt == 1 ? p.v_ts : 1.f;
  const int forced = forced_path();
  bool tc = forced != 1 && uq_verify_tc_serves(p, x);
  if (forced == 2 && !tc) return cudaErrorInvalidValue;
  cudaError_t e;
  const bool timed = t_ev_before && t_ev_after;
  if (timed) cudaEventRecord(t_ev_before, s);
  if (tc) {
    x.ns_eff = uq_verify_tc_splits(p, x);
    e = uq_verify_tc_dispatch(p, x, s);
    t_last_path = 2;
  } else {
    // enough CTAs for ~4 per SM, never more slots than the caller's scratch holds or pages exist
    const int want = std::max(1, 4 * sm_count() / std::max(1, p.B * p.HKV));
    x.ns_eff = std::max(1, std::min(std::min(p.nsplit, want), std::max(1, p.max_pages)));
    e = uq_verify_fma_dispatch(p, x, s);
    t_last_path = 1;
  }
  if (timed) cudaEventRecord(t_ev_after, s);
  if (e != cudaSuccess) return e;
  g_launches += 2;
  // (after the tcgen05 kernel, which signals its dependents at once, the combine is launched as a programmatic dependent;
  // UQ_B200_CFG="pdl=0" turns that off)
  static const bool pdl_on = !(std::getenv("UQ_B200_CFG") && std::strstr(std::getenv("UQ_B200_CFG"), "pdl=0"));
  return uq_combine_dispatch(p, x, o_part, lse_part, push, tc && pdl_on && !timed, s);
}

}  // namespace

// ---- the reference's C++ surface -------------------------------------------------------------------
// (out-of-range arguments give sizes of 2^30 rows or zero elements instead of wrapping: callers compare these with what they
// hold, and the launches refuse such arguments anyway)
int uq_block_m(int K, int HQ, int HKV) {
  if (K < 1 || HQ < 1 || HKV < 1 || K > (1 << 15) || HQ / HKV > (1 << 15)) return 1 << 30;
  return std::max(16, pow2ceil(K * pow2ceil(HQ / HKV)));
}
size_t uq_mo_elems(const UQParams& p) { return sizes_ok(p) ? (size_t)p.B * p.HKV * p.nsplit * uq_block_m(p.K, p.HQ, p.HKV) * p.D : 0; }
size_t uq_ml_elems(const UQParams& p) { return sizes_ok(p) ? (size_t)p.B * p.HKV * p.nsplit * uq_block_m(p.K, p.HQ, p.HKV) : 0; }
size_t uq_workspace_bytes(const UQParams& p) { return (uq_mo_elems(p) + uq_ml_elems(p)) * sizeof(float); }
int uq_has_sm90() { return 0; }

cudaError_t uq_decode_launch(const UQParams& p, int /*nwarps*/, int /*stages*/, cudaStream_t s) { return run(p, nullptr, nullptr, nullptr, s); }

cudaError_t uq_decode_launch_ws(UQParams p, void* workspace, int nwarps, int stages, cudaStream_t s) {
  if (!workspace) return cudaErrorInvalidValue;
  p.mo = reinterpret_cast<float*>(workspace);
  p.ml = p.mo + uq_mo_elems(p);
  return uq_decode_launch(p, nwarps, stages, s);
}

// ---- the C ABI ---------------------------------------------------------------------------------------
extern "C" {

int uqb_block_m(int K, int HQ, int HKV) { return uq_block_m(K, HQ, HKV); }
size_t uqb_mo_elems(const UQParams* p) { return uq_mo_elems(*p); }
size_t uqb_ml_elems(const UQParams* p) { return uq_ml_elems(*p); }
size_t uqb_workspace_bytes(const UQParams* p) { return uq_workspace_bytes(*p); }
int uqb_has_sm90(void) { return 0; }

int uqb_decode_launch(const UQParams* p, int nwarps, int stages, void* stream) {
  if (!p) return (int)cudaErrorInvalidValue;
  return (int)uq_decode_launch(*p, nwarps, stages, reinterpret_cast<cudaStream_t>(stream));
}

int uqb_decode_launch_ws(const UQParams* p, void* workspace, int nwarps, int stages, void* stream) {
  if (!p) return (int)cudaErrorInvalidValue;
  return (int)uq_decode_launch_ws(*p, workspace, nwarps, stages, reinterpret_cast<cudaStream_t>(stream));
}

int uqb_append_launch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const void* key, const void* value, const int64_t* slots,
                      int T, int HKV, int D, int PAGE, int dtype, void* stream) {
  return uqb_append_ex_launch(kc, ks, vc, vs, key, value, slots, T, HKV, D, PAGE, dtype, 0, 0.f, stream);
}

int uqb_append_ex_launch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const void* key, const void* value, const int64_t* slots,
                         int T, int HKV, int D, int PAGE, int dtype, int flags, float c, void* stream) {
  cudaError_t e = uq_append_dispatch(kc, ks, vc, vs, key, value, slots, T, HKV, D, PAGE, dtype, reinterpret_cast<cudaStream_t>(stream), flags, c);
  if (e == cudaSuccess && T > 0) g_launches += 1;
  return (int)e;
}

int uqb_append_nvfp4_launch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const void* key, const void* value, const int64_t* slots,
                            int T, int HKV, int D, int PAGE, int dtype, float k_ts, float v_ts, void* stream) {
  return uqb_append_nvfp4_ex_launch(kc, ks, vc, vs, key, value, slots, T, HKV, D, PAGE, dtype, k_ts, v_ts, 0, stream);
}

int uqb_append_nvfp4_ex_launch(uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, const void* key, const void* value, const int64_t* slots,
                               int T, int HKV, int D, int PAGE, int dtype, float k_ts, float v_ts, int flags, void* stream) {
  cudaError_t e = uq_append_nvfp4_dispatch(kc, ks, vc, vs, key, value, slots, T, HKV, D, PAGE, dtype, k_ts, v_ts, reinterpret_cast<cudaStream_t>(stream), flags);
  if (e == cudaSuccess && T > 0) g_launches += 1;
  return (int)e;
}

int uqb_fwht_launch(const void* x, void* out, long long rows, int D, int dtype, void* stream) {
  cudaError_t e = uq_fwht_dispatch(x, out, rows, D, dtype, reinterpret_cast<cudaStream_t>(stream));
  if (e == cudaSuccess && rows > 0) g_launches += 1;
  return (int)e;
}

int uqb_decode_partial_launch(const UQParams* p, const int32_t* pos_offset, float* o_part, float* lse2_part, void* stream) {
  if (!p || !o_part || !lse2_part) return (int)cudaErrorInvalidValue;
  return (int)run(*p, pos_offset, o_part, lse2_part, reinterpret_cast<cudaStream_t>(stream));
}

int uqb_merge_packed_launch(const float* packed, int R, size_t rows, int D, void* out_bf16, void* stream) {
  cudaError_t e = uq_merge_packed_dispatch(packed, R, rows, D, out_bf16, reinterpret_cast<cudaStream_t>(stream));
  if (e == cudaSuccess && rows > 0) g_launches += 1;
  return (int)e;
}

int uqb_tree_decode_launch(const UQParams* p, const int32_t* tree_mask, void* stream) {
  if (!p) return (int)cudaErrorInvalidValue;
  return (int)run(*p, nullptr, nullptr, nullptr, reinterpret_cast<cudaStream_t>(stream), tree_mask);
}

int uqb_merge_launch(const float* o_parts, const float* lse2_parts, int R, size_t rows, int D, void* out_bf16, void* stream) {
  cudaError_t e = uq_merge_dispatch(o_parts, lse2_parts, R, rows, D, out_bf16, reinterpret_cast<cudaStream_t>(stream));
  if (e == cudaSuccess && rows > 0) g_launches += 1;
  return (int)e;
}

int uqb_cache_to_upstream_launch(const uint8_t* kc, const uint8_t* ks, const uint8_t* vc, const uint8_t* vs, uint8_t* slots_out, long long pages, int HKV,
                                 int PAGE, int D, int slot_bytes, int flags, void* stream) {
  cudaError_t e = uq_layout_dispatch(0, const_cast<uint8_t*>(kc), const_cast<uint8_t*>(ks), const_cast<uint8_t*>(vc), const_cast<uint8_t*>(vs), slots_out, pages, HKV,
                                     PAGE, D, slot_bytes, flags, reinterpret_cast<cudaStream_t>(stream));
  if (e == cudaSuccess && pages > 0) g_launches += 1;
  return (int)e;
}

int uqb_cache_from_upstream_launch(const uint8_t* slots_in, uint8_t* kc, uint8_t* ks, uint8_t* vc, uint8_t* vs, long long pages, int HKV, int PAGE, int D,
                                   int slot_bytes, void* stream) {
  cudaError_t e = uq_layout_dispatch(1, kc, ks, vc, vs, const_cast<uint8_t*>(slots_in), pages, HKV, PAGE, D, slot_bytes, 0, reinterpret_cast<cudaStream_t>(stream));
  if (e == cudaSuccess && pages > 0) g_launches += 1;
  return (int)e;
}

// ---- context split over peer memory ---------------------------------------------------------------------------------
size_t uqb_peer_bytes(int world, size_t rows, int D) {
  if (world < 1 || world > kMaxPeers || D < 1) return 0;
  return uq_peer_total_bytes(world, uq_peer_slot_floats(rows, D));
}

int uqb_peer_alloc(size_t bytes, void** ptr, unsigned char handle64[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  if (!ptr || !handle64 || bytes == 0) return (int)cudaErrorInvalidValue;
  void* d = nullptr;
  cudaError_t e = cudaMalloc(&d, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(d, 0, bytes);   // flags and the block counter start at zero; sequence numbers start at one
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, d);
  if (e != cudaSuccess) { cudaFree(d); return (int)e; }
  std::memcpy(handle64, &h, 64);
  *ptr = d;
  return 0;
}

int uqb_peer_open(const unsigned char handle64[64], void** ptr) {
  if (!ptr || !handle64) return (int)cudaErrorInvalidValue;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

int uqb_peer_close(void* ptr) { return ptr ? (int)cudaIpcCloseMemHandle(ptr) : (int)cudaErrorInvalidValue; }
int uqb_peer_free(void* ptr) { return ptr ? (int)cudaFree(ptr) : (int)cudaErrorInvalidValue; }

int uqb_decode_partial_push_launch(const UQParams* p, const int32_t* pos_offset, void* const* bases, int world, int rank, unsigned int seq, void* stream) {
  if (!p || !bases || world < 1 || world > kMaxPeers || rank < 0 || rank >= world || seq == 0u || !sizes_ok(*p)) return (int)cudaErrorInvalidValue;
  const size_t rows = (size_t)p->B * p->K * p->HQ, slot_floats = uq_peer_slot_floats(rows, p->D);
  const int parity = (int)(seq & 1u);
  UQPeerPush push{};
  for (int r = 0; r < world; r++) {
    if (!bases[r] || !aligned(bases[r], 16)) return (int)cudaErrorInvalidValue;
    char* base = reinterpret_cast<char*>(bases[r]);
    push.slot[r] = reinterpret_cast<float*>(base) + ((size_t)parity * world + rank) * slot_floats;
    push.flag[r] = reinterpret_cast<unsigned int*>(base + uq_peer_data_bytes(world, slot_floats)) + parity * kMaxPeers + rank;
  }
  push.counter = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(bases[rank]) + uq_peer_data_bytes(world, slot_floats)) + 2 * kMaxPeers;
  push.rows_total = rows;
  push.world = world;
  push.seq = seq;
  push.raise = 1;
  return (int)run(*p, pos_offset, nullptr, nullptr, reinterpret_cast<cudaStream_t>(stream), nullptr, &push);
}

int uqb_merge_wait_launch(const void* own_base, int world, unsigned int seq, size_t rows, int D, void* out_bf16, unsigned long long wait_ns, void* stream) {
  if (seq == 0u || world < 1 || world > kMaxPeers || D < 1) return (int)cudaErrorInvalidValue;
  unsigned int* status = status_ptr();
  if (!status) return (int)cudaErrorInitializationError;
  cudaError_t e = uq_merge_wait_dispatch(own_base, world, uq_peer_slot_floats(rows, D), seq, rows, D, out_bf16, wait_ns ? wait_ns : 1000000000ull, status,
                                         reinterpret_cast<cudaStream_t>(stream));
  if (e == cudaSuccess && rows > 0) g_launches += 1;
  return (int)e;
}

int uqb_last_status(uint32_t out4[4]) {
  if (!out4) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  e = cudaMemcpyFromSymbol(out4, g_uq_status, 4 * sizeof(unsigned int));
  if (e != cudaSuccess) return (int)e;
  const unsigned int zero[4] = {0, 0, 0, 0};
  return (int)cudaMemcpyToSymbol(g_uq_status, zero, sizeof(zero));
}

size_t uqb_static_scratch_bytes(void) { return kStaticScratchFloats * sizeof(float); }

int uqb_decode_launch_static(const UQParams* p, int nwarps, int stages, void* stream) {
  if (!p) return (int)cudaErrorInvalidValue;
  if (!sizes_ok(*p)) return (int)cudaErrorInvalidValue;   // (before any size arithmetic)
  // the partials of this call must fit the built-in array: refuse, before anything is enqueued, a call that needs more
  if (uq_mo_elems(*p) + uq_ml_elems(*p) > kStaticScratchFloats) return (int)cudaErrorInvalidValue;
  {
    // every other argument check of the ordinary launch, before the device is asked for anything (the scratch pointers
    // stand in as aligned non-null values; the real ones are set below)
    UQParams probe = *p;
    probe.mo = probe.ml = reinterpret_cast<float*>(uintptr_t(256));
    if (!shape_ok(probe) || !probe.out) return (int)cudaErrorInvalidValue;
  }
  // once per device, with that device current: ask the runtime where the array lives on this device
  static std::atomic<float*> base[kMaxDevices];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  float* scratch = base[dev].load(std::memory_order_acquire);
  if (!scratch) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    scratch = reinterpret_cast<float*>(ptr);
    base[dev].store(scratch, std::memory_order_release);
  }
  UQParams q = *p;
  q.mo = scratch;
  q.ml = scratch + uq_mo_elems(q);
  return (int)uq_decode_launch(q, nwarps, stages, reinterpret_cast<cudaStream_t>(stream));
}

int uqb_last_path(void) { return t_last_path; }
void uqb_debug_events(void* before, void* after) {
  t_ev_before = reinterpret_cast<cudaEvent_t>(before);
  t_ev_after = reinterpret_cast<cudaEvent_t>(after);
}
unsigned long long uqb_launch_count(void) { return g_launches.load(); }

}  // extern "C"
