// Verify/decode attention over the paged FP4 cache on the Blackwell tensor cores (tcgen05 + TMEM).
//
// The operation is the reference's (reference cuda/uq_decode.h:1-6, oracle uqmt/attn.py:402-422); the
// kernel is built the other way round from the reference's own tcgen05 kernel
// (reference cuda/uq_decode_sm100.cuh, query rows on the 128 accumulator lanes, padded): here the KEYS
// sit on the 128 lanes and the K*G query rows are the N extent of both contractions, so tensor work is
// proportional to the rows that exist:
//     S^T[key, row] = Kdeq[key, :] . Q[row, :]        M = 128 keys, N = NT rows, K = D      (A from TMEM)
//     O^T[d,   row] += Vdeq[key, d] * P[key, row]     M = 128 channels, N = NT rows, K = 128 keys
//
// head_dim 128 with the UltraQuant cache takes S^T from a block-scaled contraction (kind::mxf8f6f4, one UE8M0 scale per 32
// channels = the cache's own format): the K codes are never decoded (the copy engine unpacks them, the scale bytes go to
// TMEM as they are) and Q is two e4m3 tiles (leading bits + remainder).  head_dim 64 / 256 and the NVFP4 cache decode K to
// fp16 into a TMEM A operand instead.
//
// One CTA per SM, persistent over a flat list of 128-key tiles.  Warp roles (NSG = 4 softmax warpgroups at 32+ rows, else 2):
//   softmax   4*NSG warps  thread = (key, NT/NSG rows): reads its lane of S^T from TMEM, exp2 against a per-row REFERENCE
//                          that is fixed at the segment's first tile (quick pass; a segment where a probability or V value
//                          then overflows fp16 is found by its epilogue and run again on the careful path, where the threads
//                          agree tile by tile on moving the references), writes P^T fp16 (MN-major B operand) times the key's
//                          V reference relative to the segment's, keeps row sums in registers; at the end of a segment
//                          reduces the sums, reads O^T and writes the normalised partial with m + log2 l.
//   relay     4 warps      block-scaled: the tile's K scale bytes -> TMEM, the keys' largest V scale bytes -> a side band for
//                          the softmax threads.  Otherwise these are the K decode warps (thread = key: e2m1 -> fp16 by the
//                          hardware conversion, one fp16 multiply by the group scale relative to the key's largest,
//                          tcgen05.st into the TMEM A operand).
//   V decode  4 warps at 64 rows, 8 below (two groups that take turns at the tiles): thread = key, the same decode ->
//                          128-byte-swizzled fp16 tile in shared memory (ring of 2); gives its raw stage back as soon as the
//                          key's codes and scale bytes are in registers.
//   copy      2 warps      (K side / V side of every tile) TMA tensor copies of the code pages + bulk copies of the scale
//                          pages into a ring of raw stages (3 at head_dim 128), mbarrier complete_tx.  No multicast.
//   issue     1 thread     chosen by elect.sync: P.V of tile i, then Q.K of tile i + 2; tcgen05.commit to mbarriers; owns the
//                          TMEM allocation.
// Work is a flat list of tiles over all (sequence, kv head) items, cut into chunks of equal WEIGHT (an item counts its tiles
// plus a few for what a segment start costs), one per CTA; a chunk that crosses items yields several segments, each written
// to its own partial slot.  One warp works the CTA's segments out at set-up (a candidate item per lane) and every role
// reads them from shared memory.
//
// Every wait is bounded (about one second): on expiry the thread records the barrier in the status record, raises the CTA's
// abort flag and every role drains to the common exit, which frees TMEM.
//
// Where the time goes (headline shape, K=8, B200): the call is bound neither by HBM (the same call on an L2-resident cache is
// 3 % faster), nor by the tensor pipe (without its instructions: 2 % faster), but by the roles' serial chains: with every
// role reduced to its waits and arrivals and the tensor instructions left out, the copy ring and the hand-shakes alone take
// 91 us against 122 for the whole call.  Per CTA the time is 0.85 us per tile (1 660 cycles; the four V-decode warps are the
// longest role: 1 210 cycles of decode, 450 between tiles) plus about 25 us that do not depend on the context: set-up,
// the first segment's query conversion and first tile (which fixes the references), the epilogue, and the spread of the
// CTAs' finishing times.
#include <cuda.h>

#include <algorithm>
#include <atomic>

#include "uq_common.cuh"

namespace tc {

__device__ __forceinline__ unsigned long long now_ns_early() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

#ifdef UQ_TC_TRACE
// timeline of CTA 0 (developer build only): clock64 stamps of each role's events for its first 64 tiles
__device__ long long g_tc_trace[64][16];
#ifndef UQ_TRACE_CTA
#define UQ_TRACE_CTA 0
#endif
#ifndef UQ_TRACE_FROM
#define UQ_TRACE_FROM 0
#endif
#define UQ_TRACE(ev, c) if (blockIdx.x == UQ_TRACE_CTA && (c) >= UQ_TRACE_FROM && (c) < UQ_TRACE_FROM + 64) g_tc_trace[(c) - UQ_TRACE_FROM][ev] = clock64();
// per-CTA milestones (global timer, ns): 0 entry, 1 set-up done, 2 first tile's softmax done, 3 last tile's softmax done, 4 exit, 5 tiles, 6 segments
__device__ unsigned long long g_tc_cta[160][8];
#define UQ_TRACE_CTA_T(i) if (threadIdx.x == 0 && blockIdx.x < 160) g_tc_cta[blockIdx.x][i] = now_ns_early();
#define UQ_TRACE_CTA_V(i, v) if (threadIdx.x == 0 && blockIdx.x < 160) g_tc_cta[blockIdx.x][i] = (unsigned long long)(v);
// stamps of the softmax role's steps around a change of segment (rows 60-63 of the same table, one row per segment)
#define UQ_TRACE_SEG(ev) if (blockIdx.x == UQ_TRACE_CTA && st == 0 && seg_i < 4) g_tc_trace[60 + seg_i][ev] = clock64();
#else
#define UQ_TRACE(ev, c)
#define UQ_TRACE_SEG(ev)
#define UQ_TRACE_CTA_T(i)
#define UQ_TRACE_CTA_V(i, v)
#endif
#ifdef UQ_TC_PROF
// per-role cycle counters (profiling build only): [role][0..5] cycles spent in the role's wait sites, [6] event count, [7] total cycles
__device__ unsigned long long g_tc_prof[5][8];
#define UQ_PROF_DECL unsigned long long pw[8] = {0, 0, 0, 0, 0, 0, 0, 0}; const long long pt0 = clock64();
#define UQ_PROF_FLUSH(role, leader) if (leader) { pw[7] = clock64() - pt0; for (int i = 0; i < 8; i++) atomicAdd(&g_tc_prof[role][i], pw[i]); }
#define UQ_PROF_SITE(n) , &pw[n]
#define UQ_PROF_COUNT(n) pw[n]++;
#define UQ_PROF_T0 const long long ps0 = clock64();
#define UQ_PROF_T1(n) pw[n] += clock64() - ps0;
#define UQ_PROF_TA long long psa = clock64();
#define UQ_PROF_TA2 psa = clock64();
#define UQ_PROF_TB(n) { const long long psb = clock64(); pw[n] += psb - psa; psa = psb; }
#else
#define UQ_PROF_DECL
#define UQ_PROF_FLUSH(role, leader)
#define UQ_PROF_SITE(n) , nullptr
#define UQ_PROF_COUNT(n)
#define UQ_PROF_T0
#define UQ_PROF_T1(n)
#define UQ_PROF_TA
#define UQ_PROF_TA2
#define UQ_PROF_TB(n)
#endif

#ifndef UQ_RS128
#define UQ_RS128 3   // raw tiles in flight at head_dim 128
#endif
#ifndef UQ_SB128
#define UQ_SB128 3   // K / S^T / P^T ring depth at head_dim 128
#endif
#ifndef UQ_PROD2
#define UQ_PROD2 1   // copy warps beside the first: 0 one warp issues everything; 1 K side / V side; 2 K codes / V codes / both scale slices
#endif
#ifndef UQ_QKMERGE
#define UQ_QKMERGE 32   // block-scaled Q.K with up to this many rows: the leading and the remainder tile of Q are ONE B operand of 2 NT rows (half the Q.K instructions; the softmax adds the two halves of S^T); 0 = never
#endif
#ifndef UQ_EARLY
#define UQ_EARLY 1   // 1: the V decode gives its raw stage back once the tile's codes are in registers, not after the decode
#endif
#ifndef UQ_V64
#define UQ_V64 4   // V-decode warps at 64 rows
#endif
#ifndef UQ_NSG4_AT
#define UQ_NSG4_AT 32
#endif
#ifndef UQ_ABL
#define UQ_ABL 0   // timing experiments only (results become wrong): 1 no exp2, 2 no P write, 4 no reference loads, 8 no score loads, 16 no work in the softmax's common tile, 32 no V decode, 64 no scale relay, 128 / 256 / 512 softmax / V / relay reduced to their waits and arrivals, 1024 no tensor instructions (commits only), 2048 no copies of the scale slices
#endif
constexpr int kKeys = 128;      // keys per tile = accumulator lanes
// Thread layout: NSG softmax warpgroups (each owns NT / NSG query rows of every key), then K decode (4 warps), V decode (4),
// producer, Q.K issue, P.V issue, one idle warp.  The roles are latency bound (one warp of a role per SM sub-partition issues
// about once per 10 cycles), so the softmax, the longest role at 64 rows, is spread over four warpgroups.
__host__ __device__ constexpr int softmax_groups(int NT) { return NT >= UQ_NSG4_AT ? 4 : 2; }
// With fewer than 64 rows the V decode is the longest role and the CTA has warps to spare: eight V warps, each thread
// half of its key's scale groups; with 64 rows the softmax is, and issue slots are what it lacks: four V warps.
__host__ __device__ constexpr int v_warps(int NT) { return NT < 64 ? 8 : UQ_V64; }
__host__ __device__ constexpr int cta_threads(int NT) { return (4 * softmax_groups(NT) + 8 + v_warps(NT)) * 32; }
// ring depths; head_dim 256 doubles every tile, so its rings are shallower (512 TMEM columns, 227 KB of shared memory)
__host__ __device__ constexpr bool block_scaled(int D) { return D == 128; }          // Q.K straight from the e2m1 codes and scale bytes (see Cfg::kBS)
#ifndef UQ_RS128_16
#define UQ_RS128_16 4   // raw tiles in flight at head_dim 128 with up to 16 rows
#endif
#ifndef UQ_RS128_32
#define UQ_RS128_32 3   // ... with up to 32 rows (the P^T tiles of fewer rows share buffers: room for more raw stages)
#endif
#ifndef UQ_PSHARE
#define UQ_PSHARE 1     // 1: P^T tiles of 16 / 32 rows sit side by side in one 64-row buffer (four / two ring slots per buffer)
#endif
// raw code/scale tiles in flight (TMA)
__host__ __device__ constexpr int raw_stages(int D, int NT) { return D == 256 ? 2 : (D == 128 ? (NT <= 16 ? UQ_RS128_16 : (NT <= 32 ? UQ_RS128_32 : UQ_RS128)) : 4); }
#ifndef UQ_SB128_16
#define UQ_SB128_16 3   // the same ring at head_dim 128 with up to 16 rows
#endif
#ifndef UQ_SB128_32
#define UQ_SB128_32 3   // ... with up to 32 rows
#endif
// K operand (TMEM), S^T accumulators (TMEM), P^T tiles (shared memory); at most 4 deep (barrier indices)
__host__ __device__ constexpr int ring_sb(int D, int NT) { return D == 256 ? 2 : (D == 128 ? (NT <= 16 ? UQ_SB128_16 : (NT <= 32 ? UQ_SB128_32 : UQ_SB128)) : 3); }
__host__ __device__ constexpr int ring_vb(int D) { return D == 256 ? 1 : 2; }      // decoded V tiles (shared memory)
constexpr float kRescaleAt = 12.0f;  // a score this far (log2) above the row's reference maximum does not fit the fp16 probability tile
constexpr int kRedoWords = 32;       // a CTA's first 32 * kRedoWords segments can be marked for the second pass; later ones take the careful path at once
constexpr float kNegBig = -1.0e30f;

// ---------------------------------------------------------------------------------------------- PTX
UQ_DEV uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
UQ_DEV void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
UQ_DEV void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
UQ_DEV void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
// One blocking try: the thread is suspended by the hardware until the phase completes or the time hint (nanoseconds)
// runs out.  Without the hint a failed try returns almost at once, and several waiting warps then spin through the
// issue slots the working warps of their sub-partition need.
UQ_DEV uint32_t mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000000u) : "memory");
  return ok;
}
// Non-blocking test of a phase: about a third of the cost of a blocking try when the phase is already complete, which is
// the common case for most waits of this kernel.
UQ_DEV uint32_t mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
UQ_DEV unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// One lane of the (converged) warp: the compiler knows the guarded region runs in a single thread and can keep its
// addresses and descriptors on the uniform datapath.
UQ_DEV bool elect_one() {
  uint32_t r;
  asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(r));
  return r != 0;
}
UQ_DEV void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
UQ_DEV void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
UQ_DEV void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
UQ_DEV void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
UQ_DEV void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
UQ_DEV void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
UQ_DEV void tc_commit(uint32_t bar) { asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory"); }

// The cache is read once per call and is larger than L2: its lines are marked "evict first", so that streaming it does not
// push out what every call comes back to (the queries, the page table, the partials the combine kernel reads, the kernel's
// own instructions).
#ifndef UQ_EVICT_FIRST
#define UQ_EVICT_FIRST 1
#endif
UQ_DEV uint64_t l2_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
// 2-D tiled TMA load: box (inner 0.., rows y..) of the tensor map into shared memory, bytes counted on `bar`.
UQ_DEV void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar, uint64_t pol) {
  if (UQ_EVICT_FIRST)
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar), "l"(pol) : "memory");
  else
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// contiguous bulk copy (scale pages)
UQ_DEV void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t pol) {
  if (UQ_EVICT_FIRST)
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol) : "memory");
  else
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// shared-memory matrix descriptor, 128-byte swizzle (sm_100 format: version bit 46, layout type 2 at bit 61)
UQ_DEV uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor, kind::f16: bf16 x bf16 -> fp32; major 0 = K-major, 1 = MN-major
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, int a_mn_major, int b_mn_major, int a_bf16 = 1, int b_bf16 = 1) {
  return (1u << 4) | ((uint32_t)a_bf16 << 7) | ((uint32_t)b_bf16 << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
UQ_DEV void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// block-scaled form (kind::mxf8f6f4, UE8M0 scales, one per 32 elements of K): the scale bytes sit in TMEM, lane l of every
// 32-lane quarter, column j, byte id = row 32 j + l's scale for the instruction whose descriptor names byte `id`
UQ_DEV void mma_bs(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %6, 0;\n tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate) : "memory");
}
// its instruction descriptor: B scale byte id [4,6), A format [7,10) and B format [10,13) (0 = e4m3, 5 = e2m1), both K-major,
// N >> 3 at [17,23), UE8M0 scales (bit 23), M >> 4 at [24,29), A scale byte id [29,31)
__host__ __device__ constexpr uint32_t instr_desc_bs(int M, int N, int a_fmt, int b_fmt, int a_sf, int b_sf) {
  return ((uint32_t)b_sf << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(N >> 3) << 17) | (1u << 23) | ((uint32_t)(M >> 4) << 24) | ((uint32_t)a_sf << 29);
}
UQ_DEV void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
UQ_DEV void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
                 "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr) : "memory");
}
UQ_DEV void tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr) : "memory");
}
UQ_DEV void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
UQ_DEV void tmem_st4(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}
UQ_DEV void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
                 "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
UQ_DEV float fast_exp2(float v) {   // 2^v, -inf -> 0
  float d;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(d) : "f"(v));
  return d;
}
// packed fp32 pairs: one issue slot for two operations (the kernel is short of issue slots, not of FMA-pipe cycles)
UQ_DEV void fma_f32x2(float& d0, float& d1, float a0, float a1, float b, float c0, float c1) {   // d = a * b + c
  asm("{\n .reg .b64 ra, rb, rc, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %4};\n mov.b64 rc, {%5, %6};\n fma.rn.f32x2 rd, ra, rb, rc;\n mov.b64 {%0, %1}, rd;\n}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c0), "f"(c1));
}
UQ_DEV void add_f32x2(float& d0, float& d1, float a0, float a1) {   // d += a
  asm("{\n .reg .b64 ra, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rd, {%0, %1};\n add.rn.f32x2 rd, rd, ra;\n mov.b64 {%0, %1}, rd;\n}"
      : "+f"(d0), "+f"(d1) : "f"(a0), "f"(a1));
}
UQ_DEV uint32_t mul_f16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
UQ_DEV uint32_t pack_f16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
// two floats -> e4m3 pair (low byte = lo), saturating; and back
UQ_DEV uint32_t pack_e4m3x2(float lo, float hi) {
  unsigned short d;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
  return d;
}
UQ_DEV void unpack_e4m3x2(uint32_t v, float& lo, float& hi) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((unsigned short)v));
  lo = __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu)));
  hi = __half2float(__ushort_as_half((unsigned short)(h2 >> 16)));
}
UQ_DEV uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

// Wait for phase `parity` of an mbarrier, for about one second at most.  false = gave up (this thread's wait ran
// out, or another thread of the CTA raised the abort flag): the caller leaves its loop and falls through to the exit.
__device__ __noinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned int* status, int id, int tile) {
  const unsigned long long t_start = now_ns();
  for (unsigned it = 1;; it++) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag) return false;
      if (now_ns() - t_start > 1000000000ull) {
        *abort_flag = 1;
        uq_report(status, 1u, (unsigned)id, (unsigned)tile);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- decode
// One cvt per code byte gives the byte's two channels as an exact fp16 pair in natural order (low nibble = even channel),
// zero and sign included; one fp16 multiply applies the group scale RELATIVE to the key's largest group scale,
// 2^(s_g - ref) <= 1 (exact down to 2^-24, zero below: such a group is under 2^-24 of the key's largest).  The key's
// reference 2^(ref - 127) is applied in fp32 by the softmax threads that own the key: K's to the score, V's to the
// probability.  Both operands of a tcgen05.mma kind::f16 must have the same 16-bit format on this hardware (an fp16 A
// with a bf16 B raised "illegal instruction"), so Q and P are fp16 as well; accumulators are fp32.
UQ_DEV void decode8_f16(uint32_t w, uint32_t mult, uint32_t* out) {
  uint32_t a, b, c, d;
  asm("{\n .reg .b8 t0, t1, t2, t3;\n mov.b32 {t0, t1, t2, t3}, %4;\n cvt.rn.f16x2.e2m1x2 %0, t0;\n cvt.rn.f16x2.e2m1x2 %1, t1;\n"
      " cvt.rn.f16x2.e2m1x2 %2, t2;\n cvt.rn.f16x2.e2m1x2 %3, t3;\n}" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(w));
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(out[0]) : "r"(a), "r"(mult));
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(out[1]) : "r"(b), "r"(mult));
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(out[2]) : "r"(c), "r"(mult));
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(out[3]) : "r"(d), "r"(mult));
}
// 2^e (e <= 0) as an fp16 pair: normal down to 2^-14, subnormal down to 2^-24, zero below
UQ_DEV uint32_t pow2_f16x2(int e) {
  const uint32_t b = e >= -14 ? (uint32_t)(e + 15) << 10 : (e >= -24 ? 1u << (e + 24) : 0u);
  return b | (b << 16);
}
// NVFP4: two e4m3fn scale bytes (the two 16-channel blocks of a 32-channel group) as fp16 pairs.  The byte's low seven bits
// moved up by seven are an fp16 with the same mantissa and an exponent bias of 15 instead of 7: one multiply by 2^8 gives
// the value, subnormals included (exact: fp16 holds every e4m3fn value).  The code times the scale, at most 6 x 448 with
// five significant bits, is exact in fp16 as well.  (0x7f, the format's NaN, reads as 480 here; no quantiser writes it.)
UQ_DEV void e4m3_pair_f16x2(uint32_t two_bytes, uint32_t& lo, uint32_t& hi) {
  const uint32_t a = ((two_bytes & 0x80u) << 8) | ((two_bytes & 0x7Fu) << 7);
  const uint32_t b = ((two_bytes & 0x8000u)) | ((two_bytes & 0x7F00u) >> 1);
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(a | (a << 16)), "r"(0x5C005C00u));
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(b | (b << 16)), "r"(0x5C005C00u));
}
// the D/32 scale bytes of one key (2, 4 or 8 bytes, contiguous) as one 64-bit value, byte g = group g
template <int G>
UQ_DEV unsigned long long load_scales(const uint8_t* p) {
  if constexpr (G == 2) return *reinterpret_cast<const uint16_t*>(p);
  else if constexpr (G == 4) return *reinterpret_cast<const uint32_t*>(p);
  else return *reinterpret_cast<const unsigned long long*>(p);
}
template <int G>
UQ_DEV uint32_t max_byte(unsigned long long v) {
  uint32_t m = 0;
#pragma unroll
  for (int g = 0; g < G; g++) m = max(m, (uint32_t)(v >> (8 * g)) & 0xFFu);
  return m;
}
// 2^e as fp32 for any integer e (clamped to the finite range; e <= -127 uses the denormal / zero)
UQ_DEV float pow2_f32(int e) {
  e = min(e, 127);
  return e >= -126 ? __int_as_float((e + 127) << 23) : (e >= -149 ? __int_as_float(1 << (e + 149)) : 0.f);
}

// Reduction of N values per lane across the warp (N = 8 or 16), sum or maximum.  Instead of one butterfly per value
// (5 N shuffles), every step halves the values a lane still holds: lanes with the step's bit clear keep the lower half and
// take the partner's lower half, the others the upper halves: N - 1 + log2(32 / N) shuffles.  Returns the reduction of value
// warp_fold_row<N>(lane); the 32 / N lanes that differ only in their low bits hold the same value.
template <int N>
UQ_DEV int warp_fold_row(int lane) {
  int row = 0, bit = 16;
#pragma unroll
  for (int h = N / 2; h >= 1; h >>= 1, bit >>= 1) row += (lane & bit) ? h : 0;
  return row;
}
template <int N, bool kMax>
UQ_DEV float warp_fold(float* v, int lane) {
  int bit = 16;
#pragma unroll
  for (int n = N; n > 1; n >>= 1, bit >>= 1) {
    const bool hi = (lane & bit) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; i++) {
      const float give = hi ? v[i] : v[i + n / 2];
      const float keep = hi ? v[i + n / 2] : v[i];
      const float got = __shfl_xor_sync(0xffffffffu, give, bit);
      v[i] = kMax ? fmaxf(keep, got) : keep + got;
    }
  }
  float r = v[0];
#pragma unroll
  for (; bit; bit >>= 1) {
    const float got = __shfl_xor_sync(0xffffffffu, r, bit);
    r = kMax ? fmaxf(r, got) : r + got;
  }
  return r;
}

// Which of the rows r0 .. r0 + n - 1 (row = draft j * G + head of the group) see draft token td of sequence b: bit i = row
// r0 + i.  Out of line: it runs only in the one or two tiles of an item that hold the draft positions, and inlined it costs
// the common tile registers.
// (j_first: the caller's number of this launch's draft 0, K the caller's draft count, when a tree-masked call runs as chunks.)
__device__ __noinline__ uint32_t draft_rows(const int32_t* tree_mask, int K, int b, int td, int r0, int n, int rows, int G, int j_first) {
  uint32_t m = 0u;
  for (int i = 0; i < n; i++) {
    const int r = r0 + i, j = r / G + j_first;
    if (r >= rows) break;
    const bool sees = tree_mask ? ((static_cast<unsigned>(__ldg(tree_mask + (size_t)b * K + j)) >> td) & 1u) != 0u : td <= j;
    if (sees) m |= 1u << i;
  }
  return m;
}

// ---------------------------------------------------------------------------------------------- layout
struct Seg {
  int b, hk, t0, t1;   // tiles [t0, t1) of item (b, hk)
  int slot;            // partial slot of this segment
  int nseg;            // slots the item uses (valid when t0 == 0)
  int ntiles;          // tiles of the whole item
};

// A CTA's segments, worked out once at set-up by one warp (a candidate item per lane) and read by every role from shared
// memory: walking the list costs a role over a microsecond per call (an out-of-line call on a struct in local memory;
// inlined, its registers would be held across every role's tile loop), which each role used to pay before its first
// tile, between segments and once more to learn that the list had ended.
constexpr int kSegCap = 32;
struct SegList {
  int n;          // segments listed
  int more;       // 1: the CTA's chunk goes on past the listed candidates (roles continue with the walker from pos_after / it_after)
  int pos_after, it_after;
  Seg seg[kSegCap];
};

template <int D, int NT, int FMT = 0>
struct Cfg {
  static_assert(D == 64 || D == 128 || D == 256, "head_dim 64 / 128 / 256");
  static_assert(NT == 16 || NT == 32 || NT == 64, "rows padded to 16 / 32 / 64");
  static constexpr int kRawStages = raw_stages(D, NT), kSB = ring_sb(D, NT), kVB = ring_vb(D);
  static_assert(kSB <= 4, "four barrier indices per ring");
  static constexpr int kCodeRow = D / 2;                 // bytes of codes per key
  static constexpr int kGroups = D / 32;                 // 32-channel groups per key: one UE8M0 scale byte each (FMT 0)
  static constexpr int kScaleB = FMT ? D / 16 : D / 32;  // scale bytes per key (NVFP4: one e4m3fn byte per 16 channels)
  static constexpr int kChunks = kCodeRow / 16;          // 16-byte chunks per code row = scale groups
  static constexpr int kRowsPer128 = 128 / kCodeRow;     // code rows per 128 bytes: the TMA swizzle (32 / 64 / 128 B) XORs the chunk index with (row / this)
  // head_dim 128: S^T comes from a block-scaled contraction (kind::mxf8f6f4, one UE8M0 scale per 32 channels: the cache's own
  // format), so the K codes are never decoded.  The TMA unpacks them into the layout that instruction reads (16 codes = 8
  // bytes, then 8 bytes of padding: 128 bytes per key), the scale bytes go to TMEM as they are, and Q is two e4m3 tiles
  // (leading bits + remainder, each with a scale per row and 32 channels).
  static constexpr bool kBS = block_scaled(D) && FMT == 0;   // (NVFP4 scales are not powers of two: it takes the fp16 route at every head_dim)
  static constexpr int kRawCodes = kKeys * kCodeRow;
  static constexpr int kRawScales = kKeys * kScaleB;
  static constexpr int kRawK = kBS ? kKeys * D : kRawCodes;   // K codes of a tile as they sit in shared memory
  static constexpr int kOffVC = kRawK;                        // offsets within a raw stage: V codes, K scales, V scales
  static constexpr int kOffKS = kOffVC + kRawCodes;
  static constexpr int kOffVS = kOffKS + kRawScales;
  static constexpr int kRawStage = kOffVS + kRawScales;
  static_assert(!kBS || kRawStage % 1024 == 0, "the unpacked K tile is a swizzled MMA operand");
  static constexpr int kHalves = D / 64;                 // 64-channel (128-byte) column blocks of the fp16 tiles
  static constexpr int kVHalf = kKeys * 128;             // fp16 [key][64 channels]
  static constexpr int kVTile = kHalves * kVHalf;
  static constexpr int kQHalf = NT * 128;                // fp16 [row][64 channels]
  static constexpr int kQTile = kHalves * kQHalf;
  static constexpr int kPTile = kKeys * 128;             // fp16 [key][64 rows]: one 128-byte row per key, 128-byte swizzle
  // A P^T tile of NT rows fills NT * 2 bytes of every key's row: with fewer than 64 rows, kPPer ring slots sit side by side
  // in one buffer (slot s = buffer s / kPPer, 16-byte chunks (s % kPPer) * NT / 8 ...), which frees shared memory for raw stages
  static constexpr int kPPer = UQ_PSHARE ? 64 / NT : 1;
  static constexpr int kPBufs = (kSB + kPPer - 1) / kPPer;
  static constexpr int kDB = D > 128 ? D / 128 : 1;      // 128-channel blocks of O^T (one accumulator each); head_dim 64 uses the lower half of one
  // shared memory map (offsets from the 1024-aligned base)
  static constexpr int oV = 0;
  static constexpr int oQ = oV + kVB * kVTile;
  static constexpr int oP = oQ + kQTile;
  static constexpr int oRaw = oP + kPBufs * kPTile;
  static constexpr int oBar = oRaw + kRawStages * kRawStage;
  static constexpr int kNumBars = 2 * kRawStages + 24;
  static constexpr int oMisc = oBar + kNumBars * 8;
  // misc: tmem slot, abort flag, vote flags, mref[2][NT], wmax[4][NT], lsum[NT], fac[NT], facO[NT], wr[8], ref side band, prefix[]
  static constexpr int oTmemSlot = oMisc;
  static constexpr int oAbort = oMisc + 4;
  static constexpr int oVote = oMisc + 8;                // 2 ints
  static constexpr int oMref = oMisc + 16;
  static constexpr int oWmax = oMref + 2 * NT * 4;
  static constexpr int oLsum = oWmax + 4 * NT * 4;
  static constexpr int oFac = oLsum + 4 * NT * 4;        // (lsum: one partial per 32-key quarter and row, added in a fixed order)
  static constexpr int oFacO = oFac + NT * 4;            // per-row factor for O^T (row factor x V-reference factor)
  static constexpr int oWr = oFacO + NT * 4;             // [4] per-warp maxima of the keys' V reference bytes; [4..5] the segment's V reference byte (double buffered)
  static constexpr int oSfb = oWr + 32;                  // [2][NT][4] scale bytes of the two Q tiles (block-scaled path)
  static constexpr int oRef = oSfb + 2 * NT * 4;                  // [8][128] uint16: K reference byte | V reference byte << 8 of the last eight tiles (a slot is rewritten
                                                         // only after its readers, the softmax threads of a tile several ring turns back, are done)
  static constexpr int oPrefix = oRef + 8 * kKeys * 2;
  static constexpr int kMaxB = 1024;
  static constexpr int oRedo = oPrefix + (kMaxB + 1) * 4;   // kRedoWords words of per-segment "run again" bits, then one word "any bit set"
  static constexpr int oSegs = oRedo + (kRedoWords + 1) * 4;   // the CTA's first kSegCap segments (SegList), listed once at set-up
  static constexpr int kSmem = oSegs + (int)sizeof(SegList);
  static_assert(kSmem <= 227 * 1024, "shared memory budget");
  // TMEM columns
  static constexpr int kKCols = kBS ? 4 : D / 2;         // fp16 A operand of S^T: two channels per 32-bit column; block-scaled: the keys' scale bytes
  static constexpr int cK = 0;                           // kSB x kKCols
  static constexpr int cSFB = kSB * kKCols;              // block-scaled: scale bytes of the two Q tiles, 4 columns each
  static constexpr int cS = kBS ? 32 : kSB * kKCols;     // kSB x NT: fp32 S^T
  static constexpr bool kQM = kBS && NT <= UQ_QKMERGE;   // leading and remainder Q tiles contracted by one instruction: S^T = two halves of NT columns
  static constexpr int kSCols = kQM ? 2 * NT : NT;       // TMEM columns of one S^T slot
  static constexpr int cO = cS + kSB * kSCols;           // kDB x NT: fp32 O^T
  static_assert(cO + kDB * NT <= 512, "TMEM budget");
};

// barrier indices (after the raw ring's full[0..RS) and empty[0..RS))
enum { bKfull = 0, bSfull = 4, bPfull = 8, bPdone = 12, bVfull = 16, bVdone = 18, bQfull = 20, bOdone = 21, bEpi = 22, bVote = 23 };

struct Params {
  UQParams p;
  UQLaunch x;
  int chunk_min;      // lower bound on the chunk (tiles per CTA) that keeps segments per item within ns_eff
  int unit;           // tokens one copy moves: gcd(PAGE, 128) - a whole page of up to 128 tokens, a 128-token part of a larger power-of-two page, or the largest common part of a page size like 48 or 96 and the 128-key tile
};

// Position in a ring of N slots: the slot and the phase bit of the current lap, counted up tile by tile (a division and
// a remainder per tile, role and ring add up in a kernel that is bound by its instruction count).
template <int N>
struct RingPos {
  int slot;
  uint32_t phase;
  UQ_DEV void set(int cnt) { slot = cnt % N; phase = (uint32_t)(cnt / N) & 1u; }
  UQ_DEV void next() { if (++slot == N) { slot = 0; phase ^= 1u; } }
};

// ---------------------------------------------------------------------------------------------- work list

// The list is cut in WEIGHTED units: an item of n tiles counts n + kSegW, the extra units standing for what the start of
// a segment costs (query conversion, first-tile reference, epilogue), so that a CTA whose chunk crosses into a second item
// gets correspondingly fewer tiles and all CTAs finish together.  Measured from per-CTA exit times: about twelve tiles'
// time at 64 rows, eight at 32, five at 16.
#ifndef UQ_SEGW64
#define UQ_SEGW64 12
#endif
#ifndef UQ_SEGW
#define UQ_SEGW 8
#endif
#ifndef UQ_SEGW16
#define UQ_SEGW16 5    // up to 16 rows: CTAs with a second segment finished 1.7 us before the others at 8
#endif
__host__ __device__ constexpr int seg_weight(int NT) { return NT >= 64 ? UQ_SEGW64 : (NT <= 16 ? UQ_SEGW16 : UQ_SEGW); }

// n / d for a quotient known to be small (below 2^16: a CTA index, a head index): one fp32 division and a correction
// instead of the 32-bit integer division's long dependent sequence.  0 <= n < 2^31, 0 < d; the fp32 estimate is off by
// less than 2^-6 for such quotients, so at most one step either way puts it right.
UQ_DEV int small_quotient(int n, int d) {
  int q = (int)__fdividef((float)n, (float)d);
  const long long r = (long long)n - (long long)q * d;
  if (r < 0) q--;
  else if (r >= d) q++;
  return q;
}

struct Walker {
  const int* prefix;   // prefix[b] = weighted units of sequences < b (one kv head): tiles + kSegW per non-empty sequence
  int B, HKV, nitems, total, chunk, per_item, kSegW;
  int pos, end, it, cta;

  UQ_DEV void init(const int* pre, int B_, int HKV_, int ns_eff, int chunk_min, int seg_w) {
    prefix = pre; B = B_; HKV = HKV_; nitems = B * HKV; total = HKV * pre[B]; kSegW = seg_w;
    cta = blockIdx.x;
    per_item = ns_eff < 2;
    if (per_item) { it = cta - (int)gridDim.x; pos = end = 0; chunk = 1; return; }
    chunk = (total + (int)gridDim.x - 1) / (int)gridDim.x;
    if (chunk < chunk_min) chunk = chunk_min;
    if (chunk < 1) chunk = 1;
    pos = min(cta * chunk, total);
    end = min(pos + chunk, total);
    it = 0;
  }
  UQ_DEV int item_tiles(int item) const { const int b = item / HKV; return max(prefix[b + 1] - prefix[b] - kSegW, 0); }
  // Past the listed segments (out of line, like next(): the roles' loops should not carry this code or its registers)
  __device__ __noinline__ bool next_after(Seg& s, const SegList* L, bool& walking, const int* pre, int B_, int HKV_, int ns_eff, int chunk_min, int seg_w) {
    if (!walking) {
      init(pre, B_, HKV_, ns_eff, chunk_min, seg_w);
      if (per_item) it = L->it_after; else pos = min(L->pos_after, end);
      walking = true;
    }
    return next(s);
  }
  // The same walk as next(), done by one warp in one step: lane j takes the j-th candidate item from the chunk's start
  // (its item index is known without the items before it: unit position of item (b, hk) = HKV * prefix[b] + hk * width of b),
  // the lanes whose item has tiles in the chunk are the segments, in lane order.  Called after init() by all 32 lanes.
  UQ_DEV void list(SegList* L, int lane) {
    Seg s;
    bool valid = false, beyond = false;   // beyond: this candidate starts at or past the chunk's end (so do all later ones)
    if (per_item) {
      const int item = cta + lane * (int)gridDim.x;
      beyond = item >= nitems;
      if (!beyond) {
        const int n = item_tiles(item);
        if (n > 0) { s.b = item / HKV; s.hk = item - s.b * HKV; s.t0 = 0; s.t1 = n; s.slot = 0; s.nseg = 1; s.ntiles = n; valid = true; }
      }
    } else if (pos < end) {
      int lo = 0, hi = B;                 // sequence containing unit `pos`: largest b with HKV * prefix[b] <= pos
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (HKV * prefix[mid] <= pos) lo = mid; else hi = mid;
      }
      const int nv0 = prefix[lo + 1] - prefix[lo];
      const int item = lo * HKV + small_quotient(pos - HKV * prefix[lo], nv0) + lane;
      const int b = small_quotient(item, HKV), hk = item - b * HKV;
      beyond = b >= B;
      if (!beyond) {
        const int nv = prefix[b + 1] - prefix[b], n = nv - kSegW;
        const int start = HKV * prefix[b] + hk * nv, first = start + kSegW;
        beyond = start >= end;
        if (!beyond && nv > 0) {
          const int t0 = max(pos, first) - first, t1 = min(first + n, end) - first;
          if (t1 > t0) {
            const int c0 = small_quotient(first, chunk);
            s.b = b; s.hk = hk; s.ntiles = n; s.t0 = t0; s.t1 = t1; s.slot = cta - c0;
            s.nseg = small_quotient(first + n - 1, chunk) - c0 + 1;
            valid = true;
          }
        }
        if (lane == 31 && !beyond) { L->pos_after = start + nv; L->it_after = 0; }   // where a 33rd candidate would begin
      }
    } else beyond = true;
    if (per_item && lane == 31 && !beyond) { L->pos_after = 0; L->it_after = cta + 31 * (int)gridDim.x; }
    const unsigned vm = __ballot_sync(0xffffffffu, valid), bm = __ballot_sync(0xffffffffu, beyond);
    if (valid) L->seg[__popc(vm & ((1u << lane) - 1u))] = s;
    if (lane == 0) { L->n = __popc(vm); L->more = (bm >> 31) ? 0 : 1; }
  }
  __device__ __noinline__ bool next(Seg& s) {
    if (per_item) {
      for (it += (int)gridDim.x; it < nitems; it += (int)gridDim.x) {
        const int n = item_tiles(it);
        if (n == 0) continue;
        s.b = it / HKV; s.hk = it % HKV; s.t0 = 0; s.t1 = n; s.slot = 0; s.nseg = 1; s.ntiles = n;
        return true;
      }
      return false;
    }
    while (pos < end) {
      // sequence containing unit `pos`: largest b with HKV * prefix[b] <= pos
      int lo = 0, hi = B;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (HKV * prefix[mid] <= pos) lo = mid; else hi = mid;
      }
      const int nv = prefix[lo + 1] - prefix[lo];   // > 0 because pos < HKV * prefix[lo + 1]
      const int n = nv - kSegW;
      const int hk = (pos - HKV * prefix[lo]) / nv;
      const int first = HKV * prefix[lo] + hk * nv + kSegW;   // unit of the item's tile 0 (the kSegW units before it are the start-up weight)
      const int t0 = max(pos, first) - first, t1 = min(first + n, end) - first;
      if (t1 > t0) {
        s.b = lo; s.hk = hk; s.ntiles = n; s.t0 = t0; s.t1 = t1;
        const int c0 = first / chunk;   // the CTA of the item's tile 0 writes slot 0
        s.slot = cta - c0;
        s.nseg = (first + n - 1) / chunk - c0 + 1;
        pos = first + t1;
        return true;
      }
      pos = min(first + n, end);   // only start-up units of this item fall into the chunk
    }
    return false;
  }
};

// ---------------------------------------------------------------------------------------------- kernel
template <int D, int NT, int FMT>
__global__ void __launch_bounds__(cta_threads(NT), 1)
uq_verify_tc_kernel(const __grid_constant__ Params prm, const __grid_constant__ CUtensorMap map_kc, const __grid_constant__ CUtensorMap map_vc) {
  using C = Cfg<D, NT, FMT>;
  // declared 1024-byte aligned (swizzled tiles need it) and used without any integer arithmetic on the pointer, so that the
  // compiler keeps every access in the shared state space (ld.shared / st.shared instead of generic loads and stores)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  UQ_TRACE_CTA_T(0)
  // the combine kernel that follows on the stream may be set up now (its blocks wait for this grid's completion themselves)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const UQParams& p = prm.p;
  const UQLaunch& x = prm.x;
  uint8_t* sm = smem_raw;
  const uint32_t sm_a = smem_u32(sm);
  if (sm_a & 1023u) {   // never expected; the swizzled layouts below would be wrong
    if (threadIdx.x == 0) uq_report(prm.x.status, 2u, sm_a, 0u);
    return;
  }
  constexpr int NSG = softmax_groups(NT), kThreads = cta_threads(NT);
  constexpr int kRawStages = C::kRawStages, kSB = C::kSB, kVB = C::kVB;
  constexpr int kNV = v_warps(NT);
  constexpr int kWarpK = 4 * NSG, kWarpV = kWarpK + 4, kWarpProd = kWarpV + kNV, kWarpMma = kWarpProd + 1;   // first warp of each role; softmax = 0
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + C::oAbort);
  int* prefix = reinterpret_cast<int*>(sm + C::oPrefix);

  auto bar_raw_full = [&](int s) { return sm_a + C::oBar + 8 * s; };
  auto bar_raw_empty = [&](int s) { return sm_a + C::oBar + 8 * (kRawStages + s); };
  auto bar = [&](int i) { return sm_a + C::oBar + 8 * (2 * kRawStages + i); };

  // Wait on an mbarrier: a test and one blocking try inline (try_wait itself suspends the thread for a while, so these
  // almost always suffice), then the out-of-line bounded wait.  The call sits on the rare path so that the registers live across it
  // are not saved and restored on every tile.
  auto wait = [&](uint32_t b, uint32_t parity, int id, int tile, unsigned long long* site) -> bool {
#ifdef UQ_TC_PROF
    const long long c_start = clock64();
#endif
    bool r = mbar_test(b, parity);
    if (!r) r = mbar_try(b, parity);
    if (!r) r = bounded_wait(b, parity, abort_flag, x.status, id, tile);
#ifdef UQ_TC_PROF
    if (site) *site += clock64() - c_start;
#endif
    return r;
  };

  // one arrival per warp: every lane's earlier writes are ordered before it by the warp barrier
  auto warp_arrive = [&](uint32_t b) {
    __syncwarp();
    if (lane == 0) mbar_arrive(b);
  };

  // ---- set-up: barriers, tile prefix, TMEM
  if (tid == 0) {
    // a raw stage is free again after the four K (or relay) warps and the V warps have read it (block-scaled: and after the Q.K instructions have)
    for (int s = 0; s < kRawStages; s++) { mbar_init(bar_raw_full(s), UQ_PROD2 + 1); mbar_init(bar_raw_empty(s), 4 + (kNV == 8 && kVB == 2 ? 4 : kNV) + (C::kBS ? 1 : 0)); }
    // role barriers count one arrival per warp (lane 0, after __syncwarp): 128 separate arrivals per tile and
    // barrier serialise in the shared-memory unit and cost more than the work they order
    for (int i = 0; i < kSB; i++) {
      mbar_init(bar(bKfull + i), 4); mbar_init(bar(bSfull + i), 1);
      mbar_init(bar(bPfull + i), 4 * NSG); mbar_init(bar(bPdone + i), 1);
    }
    for (int i = 0; i < kVB; i++) { mbar_init(bar(bVfull + i), kNV == 8 && kVB == 2 ? 4 : kNV); mbar_init(bar(bVdone + i), 1); }
    mbar_init(bar(bQfull), 4 * NSG); mbar_init(bar(bOdone), 1); mbar_init(bar(bEpi), 4 * NSG); mbar_init(bar(bVote), 4 * NSG);
    *abort_flag = 0;
    reinterpret_cast<int*>(sm + C::oVote)[0] = 0;
    reinterpret_cast<int*>(sm + C::oVote)[1] = 0;
    fence_barrier_init();
  }
  uint32_t* redo = reinterpret_cast<uint32_t*>(sm + C::oRedo);
  for (int i = tid; i <= kRedoWords; i += kThreads) redo[i] = 0u;
  {
    // the queries (B x K x Hq x D bf16, read once per segment by whichever CTA gets it) go to L2 now, a slice per CTA, while
    // the set-up below runs: the first segment's conversion and every later one then find them there
    const size_t lines = ((size_t)p.B * p.K * p.HQ * D * 2 + 127) / 128;
    const char* qb = reinterpret_cast<const char*>(p.q);
    for (size_t i = (size_t)blockIdx.x * kThreads + tid; i < lines; i += (size_t)gridDim.x * kThreads)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(qb + i * 128));
  }
  for (int b = tid; b < p.B; b += kThreads) {   // tiles per sequence, then an in-place scan by one thread
    int off;
    const int n = uq_n_local(p, x, b, &off);
    const int tiles = (n + kKeys - 1) / kKeys;
    prefix[b + 1] = tiles ? tiles + seg_weight(NT) : 0;
  }
  __syncthreads();
  if (tid == 0) {
    prefix[0] = 0;
    for (int b = 0; b < p.B; b++) prefix[b + 1] += prefix[b];
  }
  SegList* seglist = reinterpret_cast<SegList*>(sm + C::oSegs);
  if (warp == 0) {   // the CTA's segments, once, for every role (the walker's struct lives in registers here)
    __syncwarp();
    Walker w0;
    w0.init(prefix, p.B, p.HKV, x.ns_eff, prm.chunk_min, seg_weight(NT));
    w0.list(seglist, lane);
  }
  if (warp == kWarpMma) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(sm_a + C::oTmemSlot) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(sm + C::oTmemSlot);
  UQ_TRACE_CTA_T(1)

  Walker wk;
  const int G = x.G, rows = x.rows;
  Seg sg;
  // Two passes over the CTA's segments.  The first takes every segment on the quick path: the softmax threads fix each
  // row's reference at the segment's first tile and afterwards only watch for a score or a V scale that no longer fits the
  // fp16 probability tile; a segment where that happens is marked (its result is garbage) and the second pass runs the
  // marked segments again on the careful path, where the threads agree tile by tile on moving the references.  Every role
  // walks the same list and reads the same marks, so ring slots and barrier phases simply keep counting across the passes.
  int cnt = 0, seg_i = 0;          // tiles and segments this role has processed: ring slots and barrier phases derive from them
  bool ok = true;
  int mcur = 0, nvote = 0;         // softmax role: live copy of the double-buffered references, rendezvous count
  float csc0 = x.sc2;
  for (int pass = 0; pass < 2; pass++) {
  // the listed segments first; a chunk that goes on past them (more than kSegCap candidate items: very short sequences)
  // is walked from there
  int seg_at = 0;
  bool walking = false;
  auto next_seg = [&](Seg& s) -> bool {
    if (seg_at < seglist->n) { s = seglist->seg[seg_at++]; return true; }
    if (!seglist->more) return false;
    return wk.next_after(s, seglist, walking, prefix, p.B, p.HKV, x.ns_eff, prm.chunk_min, seg_weight(NT));
  };
  int ord = -1;                    // ordinal of the segment in the CTA's list
  // does this pass run segment `ord`?  (pass 1: the marked ones)
  auto take = [&]() -> bool { ord++; return pass == 0 || (ord < 32 * kRedoWords && ((redo[ord >> 5] >> (ord & 31)) & 1u)); };

  if (warp == kWarpProd || (UQ_PROD2 >= 1 && warp == kWarpProd + 2) || (UQ_PROD2 == 2 && warp == kWarpProd + 3)) {
    // ================================================================= producer
    // what this warp copies of every tile: bit 0 K codes, bit 1 V codes, bit 2 K scales, bit 3 V scales
    const int side = (UQ_PROD2 == 0 ? 15 : (UQ_PROD2 == 1 ? (warp == kWarpProd ? 5 : 10) : (warp == kWarpProd ? 1 : (warp == kWarpProd + 2 ? 2 : 12)))) & ((UQ_ABL & 2048) ? 3 : 15);
    // a copy moves one unit: a whole page of up to 128 tokens, or a 128-token part of a larger page
    const int unit = prm.unit, ppt = kKeys / unit, spp = p.PAGE / unit;   // tokens per unit, units per tile (1 .. 8), units per page
    // (units per page are a power of two for power-of-two pages: shifts and masks then, no division in the per-tile chain)
    const bool spp_p2 = (spp & (spp - 1)) == 0;
    const int spp_sh = __ffs(spp) - 1;
    UQ_PROF_DECL
    const uint32_t page_bytes_codes = (uint32_t)unit * C::kCodeRow, page_bytes_scales = (uint32_t)unit * C::kScaleB;
    const uint64_t l2pol = l2_evict_first_policy();
    while (ok && next_seg(sg)) {
      if (!take()) continue;
      int off;
      const int n_loc = uq_n_local(p, x, sg.b, &off);
      const int pages_valid = (n_loc + unit - 1) / unit;   // (units)
      const int32_t* bt = p.block_table + (size_t)sg.b * p.max_pages;
      // Page ids come 32 units at a time, a block ahead (lane j of `cur` = unit blk0 + j, `nxt` the block after it): the
      // table's latency (an L2 round trip) stays out of the per-tile chain wait -> request.
      auto load_ids = [&](int ub) -> int { const int uu = ub + lane; return uu < pages_valid ? __ldg(bt + (spp_p2 ? uu >> spp_sh : uu / spp)) : 0; };
      int blk0 = sg.t0 * ppt;
      int cur = load_ids(blk0), nxt = load_ids(blk0 + 32);
      for (int t = sg.t0; t < sg.t1; t++, cnt++) {
        const int stage = cnt % kRawStages;
        const int vp = min(ppt, pages_valid - t * ppt);
        if (t * ppt >= blk0 + 32) { cur = nxt; blk0 += 32; nxt = load_ids(blk0 + 32); }
        // (units per tile divide 32 and blk0 is a multiple of them: a tile's units lie in one block)
        const int pid = __shfl_sync(0xffffffffu, cur, (t * ppt - blk0 + lane) & 31);
        ok = wait(bar_raw_empty(stage), ((cnt / kRawStages) & 1) ^ 1, 100 + stage, t UQ_PROF_SITE(0));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint32_t dst = sm_a + C::oRaw + stage * C::kRawStage;
        if (lane == 0) { UQ_TRACE(0, cnt) }
        if (lane == 0) mbar_expect_tx(bar_raw_full(stage), (uint32_t)vp * ((uint32_t)__popc(side & 3) * page_bytes_codes + (uint32_t)__popc(side & 12) * page_bytes_scales));
        __syncwarp();
        if (lane < vp) {
          // first cache row of this unit of (page, head); 64-bit: a cache may hold more than 2^31 / PAGE (page, head) slices
          const int in_page = spp_p2 ? (t * ppt + lane) & (spp - 1) : (t * ppt + lane) % spp;   // this unit's place in its page
          const long long row0 = ((long long)pid * p.HKV + sg.hk) * p.PAGE + in_page * unit;
          const uint32_t fb = bar_raw_full(stage);
          // block-scaled: the K map unpacks (a page lands as PAGE x 128 bytes); the bytes counted on the barrier are the packed ones
          if (side & 1) tma_load_2d(dst + lane * (C::kBS ? 2 : 1) * page_bytes_codes, &map_kc, 0, (int)row0, fb, l2pol);
          if (side & 2) tma_load_2d(dst + C::kOffVC + lane * page_bytes_codes, &map_vc, 0, (int)row0, fb, l2pol);
          if (side & 4) bulk_load(dst + C::kOffKS + lane * page_bytes_scales, p.ks + (size_t)row0 * C::kScaleB, page_bytes_scales, fb, l2pol);
          if (side & 8) bulk_load(dst + C::kOffVS + lane * page_bytes_scales, p.vs + (size_t)row0 * C::kScaleB, page_bytes_scales, fb, l2pol);
        }
      }
    }
    if (!ok) {
      // Giving up (a wait ran out somewhere in the CTA): copies this warp requested may still be in flight towards this CTA's
      // shared memory, which must not be left while they are.  Wait for the full barrier of every stage it armed, for about
      // 50 microseconds at most per stage (a copy takes one or two; a barrier whose other half was never armed cannot
      // complete, so the limit also covers the time its bytes need).
      for (int back = 0; back < kRawStages && back < cnt; back++) {
        const int c = cnt - 1 - back;
        const uint32_t fb = bar_raw_full(c % kRawStages), ph = (uint32_t)(c / kRawStages) & 1u;
        const unsigned long long t0 = now_ns();
        while (!mbar_test(fb, ph) && now_ns() - t0 < 50000ull) __nanosleep(200);
      }
    }
    UQ_PROF_FLUSH(0, lane == 0)
  } else if (warp == kWarpMma) {
    // ================================================================= MMA issue: one thread issues both contractions.
    // A tcgen05.mma with N <= 64 takes the tensor pipe about 48 cycles (its operands come from shared memory at 128 bytes a
    // cycle) when one thread issues a straight run of them; two threads issuing at once got 63 cycles per instruction between
    // them in a probe and 100-170 in this kernel.  The order is P.V of tile i, then Q.K of tile i + LA (LA = ring depth - 1):
    // S^T of the next tiles is complete before the softmax asks for it.  Everything is issued in program order and a commit
    // covers all earlier instructions of the thread, so S^T(c) complete implies P.V(c - ring depth) complete: the softmax may
    // overwrite that P^T slot without a wait of its own.
    constexpr uint32_t idesc_qk = instr_desc(128, NT, 0, 0, 0, 0);   // A = K, B = Q, both fp16 (mixed 16-bit formats are not legal)
    constexpr uint32_t idesc_pv = instr_desc(128, NT, 1, 1, 0, 0);   // A = V, B = P, both fp16
    constexpr int LA = kSB - 1;
    UQ_PROF_DECL
    // descriptors differ between instructions only in the start-address field (bits 0-13, units of 16 bytes)
    const uint64_t q_desc = smem_desc(sm_a + C::oQ, 16, 1024);
    // A = V^T: M = 128 channels = two 64-channel halves (leading-dimension offset = one half).  head_dim 64 has one half only:
    // offset 0 makes the upper 64 accumulator lanes a copy of the lower ones, which the epilogue ignores.
    const uint64_t v_desc = smem_desc(sm_a + C::oV, D == 64 ? 0 : C::kVHalf, 1024), p_desc = smem_desc(sm_a + C::oP, C::kVHalf, 1024);
    while (ok && next_seg(sg)) {
      if (!take()) continue;
      const int n = sg.t1 - sg.t0, c0 = cnt;
      if (elect_one()) {
        auto issue_qk = [&](int c) -> bool {
          const int buf = c % kSB;
          if (!wait(bar(bKfull + buf), (c / kSB) & 1, 24 + buf, c UQ_PROF_SITE(2))) return false;
          tc_fence_after();
          UQ_TRACE(5, c)
          const uint32_t d = tmem + C::cS + buf * C::kSCols, a = tmem + C::cK + buf * C::kKCols;
          if (UQ_ABL & 1024) {
            tc_commit(bar(bSfull + buf));
            if (C::kBS) tc_commit(bar_raw_empty(c % kRawStages));
          } else if constexpr (C::kBS) {
            // A = the unpacked K codes of the tile's raw stage (K-major, 128-byte rows), B = the leading and the remainder tile of Q
            const int stage = c % kRawStages;
            const uint64_t a_desc = smem_desc(sm_a + C::oRaw + stage * C::kRawStage, 16, 1024);
#pragma unroll
            for (int kb = 0; kb < D / 32; kb++) {
              if constexpr (C::kQM) {
                // one instruction over both Q tiles (rows 0 .. NT-1 the leading tile, NT .. 2 NT-1 the remainder: they are
                // contiguous in shared memory and their scale bytes are rows 0 .. 2 NT-1 of one scale operand)
                mma_bs(d, a_desc + (uint64_t)(kb * 2), q_desc + (uint64_t)(kb * 2), instr_desc_bs(128, 2 * NT, 5, 0, kb, kb), a, tmem + C::cSFB, kb ? 1u : 0u);
              } else {
                mma_bs(d, a_desc + (uint64_t)(kb * 2), q_desc + (uint64_t)(kb * 2), instr_desc_bs(128, NT, 5, 0, kb, kb), a, tmem + C::cSFB, kb ? 1u : 0u);
                mma_bs(d, a_desc + (uint64_t)(kb * 2), q_desc + (uint64_t)((C::kQHalf >> 4) + kb * 2), instr_desc_bs(128, NT, 5, 0, kb, kb), a, tmem + C::cSFB + 4, 1u);
              }
            }
            tc_commit(bar(bSfull + buf));
            tc_commit(bar_raw_empty(stage));   // the K codes of the stage have been read
          } else {
#pragma unroll
          for (int ks = 0; ks < D / 16; ks++)
            mma_ts(d, a + ks * 8, q_desc + (uint64_t)(((ks >> 2) * C::kQHalf + (ks & 3) * 32) >> 4), idesc_qk, ks ? 1u : 0u);
          tc_commit(bar(bSfull + buf));
          }
          UQ_TRACE(6, c)
          return true;
        };
        ok = wait(bar(bQfull), seg_i & 1, 30, seg_i UQ_PROF_SITE(0));
        if (ok && seg_i > 0) ok = wait(bar(bEpi), (seg_i - 1) & 1, 31, seg_i, nullptr);   // the previous segment's O^T has been read
        for (int i = 0; ok && i < LA && i < n; i++) ok = issue_qk(c0 + i);
        for (int i = 0; ok && i < n; i++) {
          const int c = c0 + i, buf = c % kSB, vb = c % kVB;
          ok = wait(bar(bPfull + buf), (c / kSB) & 1, 20 + buf, c UQ_PROF_SITE(3));
          if (ok) ok = wait(bar(bVfull + vb), (c / kVB) & 1, 22 + vb, c UQ_PROF_SITE(4));
          if (!ok) break;
          tc_fence_after();
          UQ_TRACE(7, c)
          // (a P^T slot inside a shared buffer starts (slot % kPPer) * NT rows = that many * 2 bytes into every key's row)
          const uint64_t va = v_desc + (uint64_t)(vb * (C::kVTile >> 4)), pa = p_desc + (uint64_t)((buf / C::kPPer) * (C::kPTile >> 4) + (buf % C::kPPer) * (NT * 2 >> 4));
#pragma unroll
          for (int db = 0; db < ((UQ_ABL & 1024) ? 0 : C::kDB); db++) {
#pragma unroll
            for (int kk = 0; kk < kKeys / 16; kk++)
              mma_ss(tmem + C::cO + db * NT, va + (uint64_t)((db * 2 * C::kVHalf + kk * 2048) >> 4), pa + (uint64_t)(kk * (2048 >> 4)), idesc_pv, (i == 0 && kk == 0) ? 0u : 1u);
          }
          tc_commit(bar(bPdone + buf));   // the careful path waits for it before it rescales O^T
          tc_commit(bar(bVdone + vb));
          UQ_TRACE(8, c)
          if (i + LA < n) ok = issue_qk(c + LA);
        }
        if (ok) tc_commit(bar(bOdone));
      }
      cnt = c0 + n;
      ok = __all_sync(0xffffffffu, ok);
      seg_i++;
    }
    UQ_PROF_FLUSH(1, lane == 0)
  } else if (warp >= kWarpK && warp < kWarpK + 4) {
    // ================================================================= K decode -> TMEM
    const int quad = warp & 3, kk = quad * 32 + lane;   // key of this thread = accumulator lane
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    UQ_PROF_DECL
    RingPos<kRawStages> rp;
    RingPos<kSB> sp;
    rp.set(cnt);
    sp.set(cnt);
    while (ok && next_seg(sg)) {
      if (!take()) continue;
      for (int t = sg.t0; t < sg.t1; t++, cnt++, rp.next(), sp.next()) {
        const int stage = rp.slot, buf = sp.slot;
        ok = wait(bar_raw_full(stage), rp.phase, 40 + stage, cnt UQ_PROF_SITE(0));
        if (ok && cnt >= kSB) ok = wait(bar(bSfull + buf), sp.phase ^ 1u, 44 + buf, cnt UQ_PROF_SITE(1));   // S^T of the tile that used this buffer is done: the A operand is free
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if ((UQ_ABL & 512) && cnt) { warp_arrive(bar(bKfull + buf)); warp_arrive(bar_raw_empty(stage)); continue; }
        tc_fence_after();
        if (kk == 0) { UQ_TRACE(1, cnt) }
        UQ_PROF_T0
        const uint8_t* raw = sm + C::oRaw + stage * C::kRawStage;
        // NVFP4: the block scales are bounded (e4m3fn), a key's fp16 values carry them whole and both references stay at 2^0
        unsigned long long sc = 0;
        uint32_t kref = 127u, vref = 127u;
        if constexpr (FMT == 0) {
          sc = load_scales<C::kGroups>(raw + C::kOffKS + kk * C::kGroups);
          if (!C::kBS) kref = max_byte<C::kGroups>(sc);
          vref = max_byte<C::kGroups>(load_scales<C::kGroups>(raw + C::kOffVS + kk * C::kGroups));
        }
        reinterpret_cast<uint16_t*>(sm + C::oRef)[(cnt & 7) * kKeys + kk] = (uint16_t)(kref | (vref << 8));   // for the softmax threads of this key
        if constexpr (C::kBS) {
          // block-scaled: nothing to decode.  The contraction wants the scale bytes of key 32 j + l (one 32-bit word: byte b =
          // channels 32 b ..) in column j of lane l of every 32-lane quarter: each warp writes its quarter.
          if (!(UQ_ABL & 64) || cnt == 0) {
            const uint32_t* ksw = reinterpret_cast<const uint32_t*>(raw + C::kOffKS);
            const uint32_t w4[4] = {ksw[lane], ksw[32 + lane], ksw[64 + lane], ksw[96 + lane]};
            tmem_st4(lane_addr + C::cK + buf * C::kKCols, w4);
          }
        } else {
        // the code row of this key: chunk g (16 bytes = group g) sits at chunk g ^ ((key / rows per 128 B) mod chunks) (TMA swizzle)
        const uint8_t* krow = raw + kk * C::kCodeRow;
        const int swz = (kk / C::kRowsPer128) & (C::kChunks - 1);
#pragma unroll
        for (int g0 = 0; g0 < C::kGroups; g0 += 4) {   // four groups at a time: loads first, then conversion
          constexpr int GN = C::kGroups < 4 ? C::kGroups : 4;
          uint4 c4[GN];
#pragma unroll
          for (int g = 0; g < GN; g++) c4[g] = *reinterpret_cast<const uint4*>(krow + (((g0 + g) ^ swz) << 4));
#pragma unroll
          for (int g = 0; g < GN; g++) {
            uint32_t m, m2;
            if constexpr (FMT == 0) m = m2 = pow2_f16x2((int)((uint32_t)(sc >> (8 * (g0 + g))) & 0xFFu) - (int)kref);
            else e4m3_pair_f16x2(*reinterpret_cast<const uint16_t*>(raw + C::kOffKS + kk * C::kScaleB + 2 * (g0 + g)), m, m2);
            uint32_t o[16];
            decode8_f16(c4[g].x, m, o); decode8_f16(c4[g].y, m, o + 4); decode8_f16(c4[g].z, m2, o + 8); decode8_f16(c4[g].w, m2, o + 12);
            tmem_st16(lane_addr + C::cK + buf * C::kKCols + (g0 + g) * 16, o);
          }
        }
        }
        UQ_PROF_T1(2)
        tc_wait_st();
        tc_fence_before();
        warp_arrive(bar(bKfull + buf));
        warp_arrive(bar_raw_empty(stage));
        if (kk == 0) { UQ_TRACE(2, cnt) }
        UQ_PROF_T1(3)
      }
    }
    UQ_PROF_FLUSH(2, kk == 0)
  } else if (warp >= kWarpV && warp < kWarpV + kNV) {
    // ================================================================= V decode -> shared memory (thread = key, or half a key with eight warps)
    // Eight warps with two V buffers: two groups of four take turns at the tiles (even tiles / buffer 0, odd tiles / buffer 1),
    // a thread decoding its whole key.  A role's time per tile is mostly latency (waits, fences, dependent loads), which
    // splitting a key between two threads does not shorten; two tiles in flight hide it.
    constexpr bool kAlt = kNV == 8 && kVB == 2;
    constexpr int kGPT = kAlt ? C::kGroups : C::kGroups / (kNV / 4);   // scale groups per thread
    const int vw = warp - kWarpV, kk = (vw & 3) * 32 + lane, gfirst = kAlt ? 0 : (vw >> 2) * kGPT;
    UQ_PROF_DECL
    RingPos<kRawStages> rp;
    RingPos<kVB> vp;
    rp.set(cnt);
    vp.set(cnt);
    while (ok && next_seg(sg)) {
      if (!take()) continue;
      int off;
      const int n_loc = uq_n_local(p, x, sg.b, &off);
      for (int t = sg.t0; t < sg.t1; t++, cnt++, rp.next(), vp.next()) {
        if (kAlt && (cnt & 1) != (vw >> 2)) continue;   // the other group's tile
        const int stage = rp.slot, buf = vp.slot;
        ok = wait(bar_raw_full(stage), rp.phase, 50 + stage, cnt UQ_PROF_SITE(0));
        if (ok && cnt >= kVB) ok = wait(bar(bVdone + buf), vp.phase ^ 1u, 54 + buf, cnt UQ_PROF_SITE(1));   // O^T += of the tile that used this buffer is done
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if ((UQ_ABL & 256) && cnt) { warp_arrive(bar(bVfull + buf)); warp_arrive(bar_raw_empty(stage)); continue; }
        if (vw == 0 && lane == 0) { UQ_TRACE(3, cnt) }
        UQ_PROF_T0
        const uint8_t* raw = sm + C::oRaw + stage * C::kRawStage + C::kOffVC;
        uint8_t* vt = sm + C::oV + buf * C::kVTile;
        const bool live = t * kKeys + kk < n_loc;   // keys past the end of the sequence contribute exact zeros
        unsigned long long sc = 0;
        int vref = 127;
        if constexpr (FMT == 0) {
          sc = load_scales<C::kGroups>(sm + C::oRaw + stage * C::kRawStage + C::kOffVS + kk * C::kGroups);
          vref = (int)max_byte<C::kGroups>(sc);
        }
        const uint8_t* vsc = sm + C::oRaw + stage * C::kRawStage + C::kOffVS + kk * C::kScaleB;   // (NVFP4: read per group below)
        const uint8_t* vcode = raw + kk * C::kCodeRow;
        const int swz = (kk / C::kRowsPer128) & (C::kChunks - 1);
        uint32_t vs2[kGPT];   // NVFP4: the two scale bytes of each of this thread's groups, read before the stage is given back
        if constexpr (FMT == 1) {
#pragma unroll
          for (int g = 0; g < kGPT; g++) vs2[g] = *reinterpret_cast<const uint16_t*>(vsc + 2 * (gfirst + g));
        }
#pragma unroll
        for (int gb = 0; gb < ((UQ_ABL & 32) && cnt ? 0 : kGPT); gb += 4) {
          constexpr int GN = kGPT < 4 ? kGPT : 4;
          const int g0 = gfirst + gb;
          uint4 c4[GN];
#pragma unroll
          for (int g = 0; g < GN; g++) c4[g] = *reinterpret_cast<const uint4*>(vcode + (((g0 + g) ^ swz) << 4));
          // codes and scale bytes of the tile are in registers after the last group's loads, so the raw stage can go back to
          // the copy warps now (the arrival orders the loads before it), a decode earlier than at the end
          if (UQ_EARLY && gb + 4 >= kGPT) warp_arrive(bar_raw_empty(stage));
#pragma unroll
          for (int g = 0; g < GN; g++) {
            const int gg = g0 + g;
            uint32_t m, m2;   // multiplier 0: keys past the end decode to zeros
            if constexpr (FMT == 0) m = m2 = live ? pow2_f16x2((int)((uint32_t)(sc >> (8 * gg)) & 0xFFu) - vref) : 0u;
            else {
              e4m3_pair_f16x2(vs2[gb + g], m, m2);
              if (!live) m = m2 = 0u;
            }
            uint32_t o[16];
            decode8_f16(c4[g].x, m, o); decode8_f16(c4[g].y, m, o + 4); decode8_f16(c4[g].z, m2, o + 8); decode8_f16(c4[g].w, m2, o + 12);
            // output chunk 4gg + w (8 channels) of the key's row: 64-channel half (4gg + w) >> 3, slot ((4gg + w) & 7) ^ (key & 7)
            uint8_t* vrow = vt + (gg >> 1) * C::kVHalf + kk * 128;
#pragma unroll
            for (int w = 0; w < 4; w++)
              *reinterpret_cast<uint4*>(vrow + ((((4 * gg + w) & 7) ^ (kk & 7)) << 4)) = make_uint4(o[4 * w], o[4 * w + 1], o[4 * w + 2], o[4 * w + 3]);
          }
        }
        UQ_PROF_T1(2)
        fence_async_smem();
        warp_arrive(bar(bVfull + buf));
        if (!UQ_EARLY || ((UQ_ABL & 32) && cnt)) warp_arrive(bar_raw_empty(stage));
        if (vw == 0 && lane == 0) { UQ_TRACE(4, cnt) }
        UQ_PROF_T1(3)
      }
    }
    UQ_PROF_FLUSH(3, vw == 0 && lane == 0)
  } else if (warp < 4 * NSG) {
    // ================================================================= softmax + epilogue: NSG warpgroups, NT / NSG rows each
    constexpr int HW = NT / NSG;                        // rows (columns of S^T) per thread
    constexpr int kSm = 128 * NSG;                      // threads of the role
    const int grp = warp >> 2, quad = warp & 3, kk = quad * 32 + lane, st = tid;   // st = index within the role
    const int r0 = grp * HW;                            // first row of this thread
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    float* mref = reinterpret_cast<float*>(sm + C::oMref);     // [2][NT] per-row reference maxima, live copy = mref + mcur * NT
    float* wmax = reinterpret_cast<float*>(sm + C::oWmax);     // [4][NT] per-warp row maxima of a tile (reference move only)
    float* lsum = reinterpret_cast<float*>(sm + C::oLsum);
    float* fac_s = reinterpret_cast<float*>(sm + C::oFac);     // per-row factor of a reference move, for the row sums
    float* facO_s = reinterpret_cast<float*>(sm + C::oFacO);   // the same times the V-reference factor, for O^T
    uint32_t* wr = reinterpret_cast<uint32_t*>(sm + C::oWr);   // [0..3] per-warp maxima of V reference bytes, [4 + mcur] the segment's V reference byte
    int* vote = reinterpret_cast<int*>(sm + C::oVote);
    const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(p.q);
    UQ_PROF_DECL
    auto rendezvous = [&](int id, int tile) -> bool {   // every thread of the role; orders their shared-memory traffic
      warp_arrive(bar(bVote));
      const bool r = wait(bar(bVote), nvote & 1, id, tile UQ_PROF_SITE(1));
      nvote++;
      return __all_sync(0xffffffffu, r);
    };
    auto load_scores = [&](uint32_t addr, float* dst) {
      if constexpr (HW == 8) tmem_ld8(addr, reinterpret_cast<uint32_t*>(dst));
      else {
#pragma unroll
        for (int c = 0; c < HW / 16; c++) tmem_ld16(addr + c * 16, reinterpret_cast<uint32_t*>(dst) + c * 16);
      }
      tc_wait_ld();
    };
    // S^T of this thread's rows: with the merged Q.K the sum of the slot's two halves
    auto load_s = [&](uint32_t addr, float* dst) {
      if constexpr (C::kQM) {
        float lo[HW];
        if constexpr (HW == 8) { tmem_ld8(addr, reinterpret_cast<uint32_t*>(dst)); tmem_ld8(addr + NT, reinterpret_cast<uint32_t*>(lo)); }
        else {
#pragma unroll
          for (int c = 0; c < HW / 16; c++) { tmem_ld16(addr + c * 16, reinterpret_cast<uint32_t*>(dst) + c * 16); tmem_ld16(addr + NT + c * 16, reinterpret_cast<uint32_t*>(lo) + c * 16); }
        }
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < HW; i += 2) add_f32x2(dst[i], dst[i + 1], lo[i], lo[i + 1]);
      } else load_scores(addr, dst);
    };
    auto store_cols = [&](uint32_t addr, const float* src) {
      if constexpr (HW == 8) tmem_st8(addr, reinterpret_cast<const uint32_t*>(src));
      else {
#pragma unroll
        for (int c = 0; c < HW / 16; c++) tmem_st16(addr + c * 16, reinterpret_cast<const uint32_t*>(src) + c * 16);
      }
      tc_wait_st();
    };
    // items without a single key: nobody computes them, their slots must read as empty
    for (int it = blockIdx.x; pass == 0 && it < p.B * p.HKV; it += gridDim.x) {
      { const int b = it / p.HKV; if (prefix[b + 1] - prefix[b] != 0) continue; }   // (an item with keys has tiles + the start-up weight)
      for (int i = st; i < x.ns_eff * rows; i += kSm)
        p.ml[uq_slot(p, it / p.HKV, it % p.HKV, i / rows) * x.BM + i % rows] = -INFINITY;
    }
    while (ok && next_seg(sg)) {
      if (!take()) continue;
      UQ_TRACE_SEG(0)
      const bool careful = pass == 1 || ord >= 32 * kRedoWords;
      int off;
      const int n_loc = uq_n_local(p, x, sg.b, &off);
      const int n_glob = uq_seq_len(p, x, sg.b);
      // draft positions counted back from the end: this launch's own drafts, or, for a chunk of a tree-masked call (which
      // is not cut: any query may be given any draft by its mask), all of the caller's
      const int Kq = x.tree_mask ? x.k_total : p.K, j_first = x.tree_mask ? x.k_first : 0;
      // ---- query tile in fp16, natural channel order, 128-byte swizzle, two 64-channel halves.  The tile is scaled by a
      // power of two so that its largest magnitude lies in [1, 2) (bf16 queries of any range fit fp16 this way; entries
      // below 2^-24 of the largest vanish); the power goes back into the softmax scale.
      if constexpr (C::kBS) {
        // ---- block-scaled: Q as two e4m3 tiles, Q = hi * 2^eh + lo * 2^el with one exponent pair per row and 32 channels
        // (eh puts the block's largest magnitude in [128, 256), el = eh - 5 the remainder below 256: about nine significant bits
        // relative to the block's largest entry).  A thread converts 16 channels; the two threads of a block are neighbours.
        uint8_t* sfb = sm + C::oSfb;   // [2][NT][4] scale bytes, then relayed to TMEM
        constexpr int kItems = NT * (D / 16);
        for (int i0 = 0; i0 < kItems; i0 += kSm) {
          const int i = i0 + st, n = i / (D / 16), a = i % (D / 16);
          float qv[16];
          uint32_t amax = 0;   // bf16 magnitudes compare as integers
#pragma unroll
          for (int j = 0; j < 16; j++) qv[j] = 0.f;
          if (i < kItems && n < rows) {
            const uint4* src = reinterpret_cast<const uint4*>(qg + ((uq_draft_row(x, sg.b, n / G)) * p.HQ + sg.hk * G + n % G) * D) + 2 * a;
            const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
            const uint32_t w8[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
            for (int j = 0; j < 8; j++) {
              qv[2 * j] = __uint_as_float(w8[j] << 16);
              qv[2 * j + 1] = __uint_as_float(w8[j] & 0xFFFF0000u);
              amax = max(amax, max(w8[j] & 0x7FFFu, (w8[j] >> 16) & 0x7FFFu));
            }
          }
          amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
          const int eh = max((int)(amax >> 7) - 127 - 7, -127), el = max(eh - 5, -127);
          const float sh = pow2_f32(-eh), sl = pow2_f32(-el), dh = pow2_f32(eh);
          uint32_t hw[4] = {0, 0, 0, 0}, lw[4] = {0, 0, 0, 0};
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const uint32_t h = pack_e4m3x2(qv[2 * j] * sh, qv[2 * j + 1] * sh);
            float f0, f1;
            unpack_e4m3x2(h, f0, f1);
            const uint32_t l = pack_e4m3x2((qv[2 * j] - f0 * dh) * sl, (qv[2 * j + 1] - f1 * dh) * sl);
            hw[j >> 1] |= h << (16 * (j & 1));
            lw[j >> 1] |= l << (16 * (j & 1));
          }
          if (i < kItems) {
            const int o = n * 128 + ((a ^ (n & 7)) << 4);
            *reinterpret_cast<uint4*>(sm + C::oQ + o) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            *reinterpret_cast<uint4*>(sm + C::oQ + C::kQHalf + o) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
            if (!(a & 1)) { sfb[n * 4 + (a >> 1)] = (uint8_t)(eh + 127); sfb[(NT + n) * 4 + (a >> 1)] = (uint8_t)(el + 127); }
          }
        }
        UQ_TRACE_SEG(1)
        ok = rendezvous(59, seg_i);
        UQ_TRACE_SEG(2)
        if (!ok) break;
        if (grp == 0) {   // one warp per 32-lane quarter: the scale bytes of row 32 j + l go to column j of lane l
          const uint32_t* sw = reinterpret_cast<const uint32_t*>(sfb);
          uint32_t h4[4], l4[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const int row = 32 * j + lane;
            if constexpr (C::kQM) {   // one scale operand of 2 NT rows: the leading tile's rows, then the remainder's
              h4[j] = row < 2 * NT ? sw[row] : 0x7F7F7F7Fu;
              l4[j] = 0x7F7F7F7Fu;
            } else {
              h4[j] = row < NT ? sw[row] : 0x7F7F7F7Fu;
              l4[j] = row < NT ? sw[NT + row] : 0x7F7F7F7Fu;
            }
          }
          tmem_st4(lane_addr + C::cSFB, h4);
          if (!C::kQM) tmem_st4(lane_addr + C::cSFB + 4, l4);
          tc_wait_st();
        }
        tc_fence_before();
        csc0 = x.sc2;
      } else {
        uint32_t amax = 0;   // bf16 magnitudes compare as integers
        for (int i = st; i < rows * (D / 8); i += kSm) {
          const int n = i / (D / 8), a = i % (D / 8);
          const uint4 v = __ldg(reinterpret_cast<const uint4*>(qg + ((uq_draft_row(x, sg.b, n / G)) * p.HQ + sg.hk * G + n % G) * D) + a);
          const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; j++) amax = max(amax, max(w4[j] & 0x7FFFu, (w4[j] >> 16) & 0x7FFFu));
        }
        amax = __reduce_max_sync(0xffffffffu, amax);
        if (lane == 0) reinterpret_cast<uint32_t*>(wmax)[warp] = amax;
        ok = rendezvous(59, seg_i);
        if (!ok) break;
        const uint32_t* wq = reinterpret_cast<const uint32_t*>(wmax);
        amax = 0;
#pragma unroll
        for (int w = 0; w < 4 * NSG; w++) amax = max(amax, wq[w]);
        int eq = amax ? (int)(amax >> 7) - 127 : 0;
        eq = min(max(eq, -126), 126);
        const float qf = __int_as_float((127 - eq) << 23);
        csc0 = x.sc2 * __int_as_float((127 + eq) << 23);
        for (int i = st; i < NT * (D / 8); i += kSm) {
          const int n = i / (D / 8), a = i % (D / 8);
          uint4 w = make_uint4(0, 0, 0, 0);
          if (n < rows) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(qg + ((uq_draft_row(x, sg.b, n / G)) * p.HQ + sg.hk * G + n % G) * D) + a);
            w.x = pack_f16x2(__uint_as_float(v.x << 16) * qf, __uint_as_float(v.x & 0xFFFF0000u) * qf);
            w.y = pack_f16x2(__uint_as_float(v.y << 16) * qf, __uint_as_float(v.y & 0xFFFF0000u) * qf);
            w.z = pack_f16x2(__uint_as_float(v.z << 16) * qf, __uint_as_float(v.z & 0xFFFF0000u) * qf);
            w.w = pack_f16x2(__uint_as_float(v.w << 16) * qf, __uint_as_float(v.w & 0xFFFF0000u) * qf);
          }
          *reinterpret_cast<uint4*>(sm + C::oQ + (a >> 3) * C::kQHalf + n * 128 + (((a & 7) ^ (n & 7)) << 4)) = w;
        }
      }
      // padding rows (no query behind them) get a reference of +1e30: their probabilities are 2^-inf = 0 without a select
      if (st < NT) { mref[mcur * NT + st] = st < rows ? kNegBig : 1.0e30f; }
      if (st == 0) wr[4 + mcur] = 0u;
      fence_async_smem();
      // (test of the give-up path: with expire_id 30 the query tile is never announced, so the issuing thread's wait for it,
      // barrier id 30, really runs out after its second; the comparison sits here, once per segment, not in the per-tile waits)
      if (x.expire_id != 30) warp_arrive(bar(bQfull));
      UQ_TRACE_SEG(3)
      // the first segment of an item marks the slots the item does not use as empty
      if (sg.t0 == 0)
        for (int i = st; i < (x.ns_eff - sg.nseg) * rows; i += kSm)
          p.ml[uq_slot(p, sg.b, sg.hk, sg.nseg + i / rows) * x.BM + i % rows] = -INFINITY;
      // (no rendezvous here: the first tile reads none of these before the rendezvous of its reference move)
      UQ_TRACE_SEG(4)
      float l[HW];
#pragma unroll
      for (int i = 0; i < HW; i++) l[i] = 0.f;
      const int c0 = cnt;
      // tiles from this index on need masks (they reach the end of the sequence or the draft positions); the others are
      // the common tiles
      int tmask;
      {
        const int xq = n_glob - Kq - off - (kKeys - 1) - (x.tree_mask ? 1 : 0);
        tmask = min(n_loc / kKeys, xq < 0 ? 0 : xq / kKeys + 1);
      }
      for (int t = sg.t0; ok && t < sg.t1; t++, cnt++) {
        if (!careful && cnt > c0 && t < tmask) {
          // ---- a run of common tiles of the quick path: references fixed, no masks, nothing to agree on.  The loop keeps
          // only what such a tile needs (the kernel is bound by the number of instructions per tile): ring slot
          // and phase are counted up instead of divided out, per-segment values are read once.
          const int t_end = min(sg.t1, tmask);
          int buf = cnt % kSB;
          uint32_t sph = (uint32_t)(cnt / kSB) & 1u;
          const float4* m4 = reinterpret_cast<const float4*>(mref + mcur * NT + r0);   // fixed for the run
          const int rbyte = (int)wr[4 + mcur];
          const uint16_t* oref = reinterpret_cast<const uint16_t*>(sm + C::oRef) + kk;
          uint8_t* pk = sm + C::oP + kk * 128;
          for (; t < t_end; t++, cnt++) {
            bool r = wait(bar(bSfull + buf), sph, 62 + buf, cnt UQ_PROF_SITE(0));
            r = __all_sync(0xffffffffu, r);
            if (!r) { ok = false; break; }
            if (UQ_ABL & 128) { warp_arrive(bar(bPfull + buf)); if (++buf == kSB) { buf = 0; sph ^= 1u; } continue; }
            tc_fence_after();
            if (st == 0) { UQ_TRACE(9, cnt) }
            float pv[HW];
            load_s(lane_addr + C::cS + buf * C::kSCols + r0, pv);
            const uint32_t rf = oref[(cnt & 7) * kKeys];
            const float nck = C::kBS ? -csc0 : -(csc0 * uq_scale_f32(rf & 0xFFu));
            const uint32_t vf = pow2_f16x2(min((int)(rf >> 8) - rbyte, 16));
            if (st == 0) { UQ_TRACE(10, cnt) }
#pragma unroll
            for (int j = 0; j < HW / 4; j++) {   // 2^(s * ck - m) as 2^-(s * (-ck) + m), two rows per fused multiply-add
              const float4 m = m4[j];
              float y0, y1, y2, y3;
              fma_f32x2(y0, y1, pv[4 * j], pv[4 * j + 1], nck, m.x, m.y);
              fma_f32x2(y2, y3, pv[4 * j + 2], pv[4 * j + 3], nck, m.z, m.w);
              pv[4 * j] = fast_exp2(-y0); pv[4 * j + 1] = fast_exp2(-y1); pv[4 * j + 2] = fast_exp2(-y2); pv[4 * j + 3] = fast_exp2(-y3);
            }
            uint8_t* pt = pk + (buf / C::kPPer) * C::kPTile;
            const int pc0 = (buf % C::kPPer) * (NT / 8) + r0 / 8;   // first 16-byte chunk of this thread's rows in the key's row
#pragma unroll
            for (int c = 0; c < HW / 8; c++)
              *reinterpret_cast<uint4*>(pt + (((pc0 + c) ^ (kk & 7)) << 4)) =
                  make_uint4(mul_f16x2(pack_f16x2(pv[8 * c], pv[8 * c + 1]), vf), mul_f16x2(pack_f16x2(pv[8 * c + 2], pv[8 * c + 3]), vf),
                             mul_f16x2(pack_f16x2(pv[8 * c + 4], pv[8 * c + 5]), vf), mul_f16x2(pack_f16x2(pv[8 * c + 6], pv[8 * c + 7]), vf));
            if (st == 0) { UQ_TRACE(11, cnt) }
#pragma unroll
            for (int i = 0; i < HW; i += 2) add_f32x2(l[i], l[i + 1], pv[i], pv[i + 1]);
            tc_fence_before();
            fence_async_smem();
            warp_arrive(bar(bPfull + buf));
            if (st == 0) { UQ_TRACE(13, cnt) }
            UQ_TRACE_CTA_T(3)
            if (++buf == kSB) { buf = 0; sph ^= 1u; }
          }
          if (!ok || t >= sg.t1) break;
        }
        const int buf = cnt % kSB;
        ok = wait(bar(bSfull + buf), (cnt / kSB) & 1, 62 + buf, cnt UQ_PROF_SITE(0));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (st == 0) { UQ_TRACE(9, cnt) }
        UQ_PROF_TA
        const uint32_t s_addr = lane_addr + C::cS + buf * C::kSCols + r0;
        // this key: reference scale bytes, position, visibility
        const uint32_t rf = reinterpret_cast<const uint16_t*>(sm + C::oRef)[(cnt & 7) * kKeys + kk];
        const int vref = (int)(rf >> 8);
        const float ck = C::kBS ? csc0 : csc0 * uq_scale_f32(rf & 0xFFu);   // block-scaled scores carry the keys' scales already
        // only a tile that reaches the end of the sequence or the draft positions needs masks (same answer in every thread)
        // (chain: draft token 0 is seen by every row, so the masks start at draft 1; a tree may hide draft 0 from some rows)
        const bool need_mask = t * kKeys + kKeys - 1 >= n_loc || off + t * kKeys + kKeys - 1 + (x.tree_mask ? 1 : 0) > n_glob - Kq;
        bool live = true;
        uint32_t vmask = 0xFFFFFFFFu;   // bit i: row r0 + i sees this key
        if (need_mask) {
          const int key = t * kKeys + kk;
          live = key < n_loc;
          const int td = off + key - (n_glob - Kq);   // >= 0: the key is draft token td
          if (!live) vmask = 0u;
          else if (td >= 0) vmask = draft_rows(x.tree_mask, Kq, sg.b, td, r0, HW, rows, G, j_first);
        }
        uint8_t* pt = sm + C::oP + (buf / C::kPPer) * C::kPTile + kk * 128;
        const int pc0 = (buf % C::kPPer) * (NT / 8) + r0 / 8;
        float pv[HW];
        // scores -> probabilities against the references `mrow`, in place, with the masks; returns the largest exponent seen
        // (the form for masked tiles, first tiles and the careful path; the common tile has a leaner one below)
        auto probabilities = [&](const float* mrow) -> float {
          float xm = kNegBig;
#pragma unroll
          for (int i = 0; i < HW; i++) {
            float xv = fmaf(pv[i], ck, (UQ_ABL & 4) ? -1.0f : -mrow[r0 + i]);
            xm = fmaxf(xm, xv);
            pv[i] = (UQ_ABL & 1) ? xv * 0.001f : fast_exp2(xv);
          }
          return xm;
        };
        // P^T row of this key: probabilities times the key's V reference relative to the segment's, fp16
        auto write_p = [&](int rbyte) {
          // the power of two is applied to the packed pairs (exact; a pair that no longer fits becomes an infinity, which the
          // votes or the epilogue see); past the end of the sequence the bytes are arbitrary: factor 0
          const uint32_t vf = live ? pow2_f16x2(min(vref - rbyte, 16)) : 0u;
#pragma unroll
          for (int c = 0; c < HW / 8; c++)
            *reinterpret_cast<uint4*>(pt + (((pc0 + c) ^ (kk & 7)) << 4)) =
                make_uint4(mul_f16x2(pack_f16x2(pv[8 * c], pv[8 * c + 1]), vf), mul_f16x2(pack_f16x2(pv[8 * c + 2], pv[8 * c + 3]), vf),
                           mul_f16x2(pack_f16x2(pv[8 * c + 4], pv[8 * c + 5]), vf), mul_f16x2(pack_f16x2(pv[8 * c + 6], pv[8 * c + 7]), vf));
        };
        // scores of a masked tile: what a row does not see becomes -inf here, once (scale factors are positive, so it stays
        // -inf; a dead key's score may be anything, NaN included)
        auto load_masked = [&]() {
          load_s(s_addr, pv);
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < HW; i++) pv[i] = ((vmask >> i) & 1u) ? pv[i] : -INFINITY;
          }
        };
        if (!(UQ_ABL & (8 | 16)) || cnt == c0) load_masked();
        else {
#pragma unroll
          for (int i = 0; i < HW; i++) pv[i] = 0.5f;
        }
        if (st == 0) { UQ_TRACE(10, cnt) }
        UQ_PROF_TB(2)
        const int rbyte = (int)wr[4 + mcur];
        const bool first = cnt == c0;              // the first tile of a segment sets the references: straight to the move below
        const bool agree = careful && !first;      // later tiles agree on a move only on the careful path
        const bool lean = !careful && !first && !need_mask;
        float xm = kNegBig;
        if (first || (lean && (UQ_ABL & 16))) {
        } else if (lean) {
          // the common tile: 2^(s * ck - m) as 2^-(s * (-ck) + m), two rows per fused multiply-add
          const float4* m4 = reinterpret_cast<const float4*>(mref + mcur * NT + r0);
          const float nck = -ck;
#pragma unroll
          for (int j = 0; j < HW / 4; j++) {
            const float4 m = m4[j];
            float y0, y1, y2, y3;
            fma_f32x2(y0, y1, pv[4 * j], pv[4 * j + 1], nck, m.x, m.y);
            fma_f32x2(y2, y3, pv[4 * j + 2], pv[4 * j + 3], nck, m.z, m.w);
            pv[4 * j] = fast_exp2(-y0); pv[4 * j + 1] = fast_exp2(-y1); pv[4 * j + 2] = fast_exp2(-y2); pv[4 * j + 3] = fast_exp2(-y3);
          }
        } else xm = probabilities(mref + mcur * NT);
        UQ_PROF_TB(3)
        if (!first && !(UQ_ABL & 2) && !((UQ_ABL & 16) && lean)) write_p(rbyte);
        if (st == 0) { UQ_TRACE(11, cnt) }
        UQ_PROF_TB(4)
        // ---- did any score leave the window of its row's reference, or any key's V scale exceed the segment's reference?
        // (the lean tiles of the quick path do not look: an overflow there leaves infinities or NaNs in O^T, which the
        // segment's epilogue finds)
        const bool grew = !lean && !first && __any_sync(0xffffffffu, xm > kRescaleAt || (live && vref > rbyte));
        const int vslot = nvote & 1;
        if (agree) {
          if (grew && lane == 0) atomicOr(&vote[vslot], 1);
          ok = rendezvous(64, cnt);
          if (!ok) break;
        } else if (!first) {
          // quick path: what this tile wrote may have overflowed; mark the segment for the second pass and carry on
          if (!UQ_ABL && grew && lane == 0) { atomicOr(&redo[ord >> 5], 1u << (ord & 31)); redo[kRedoWords] = 1u; }
        }
        if (first || (agree && *reinterpret_cast<volatile int*>(&vote[vslot]))) {
          UQ_PROF_COUNT(6)
          // ---- move the references (the first tile of a segment, then only on growth), rescale what was accumulated,
          // and redo this tile against the new references
          const float* mr = mref + mcur * NT;
          if (!first) load_masked();   // (a first tile still holds the scores it loaded)
          {
            float vv[HW];
#pragma unroll
            for (int i = 0; i < HW; i++) vv[i] = pv[i] * ck;
            const float vmax = warp_fold<HW, true>(vv, lane);
            if ((lane & (32 / HW - 1)) == 0) wmax[quad * NT + r0 + warp_fold_row<HW>(lane)] = vmax;
          }
          if (grp == 0) {
            const uint32_t vr = __reduce_max_sync(0xffffffffu, live ? (uint32_t)vref : 0u);
            if (lane == 0) wr[quad] = vr;
          }
          ok = rendezvous(65, cnt);
          if (!ok) break;
          if (st == 0) vote[0] = vote[1] = 0;
          if (st < NT) {   // thread r owns row r
            const float m_old = mr[st];
            const float m_new = fmaxf(fmaxf(m_old, fmaxf(wmax[st], wmax[NT + st])), fmaxf(wmax[2 * NT + st], wmax[3 * NT + st]));
            const int r_old = (int)wr[4 + mcur];
            const int r_new = max(max(r_old, (int)max(wr[0], wr[1])), (int)max(wr[2], wr[3]));
            const float f = fast_exp2(m_old - m_new);   // first tile: 2^(-1e30 - m) = 0
            mref[(mcur ^ 1) * NT + st] = m_new;
            fac_s[st] = f;
            facO_s[st] = f * pow2_f32(r_old - r_new);
            if (st == 0) wr[4 + (mcur ^ 1)] = (uint32_t)r_new;
          }
          ok = rendezvous(67, cnt);
          if (!ok) break;
          if (!first) {
#pragma unroll
            for (int i = 0; i < HW; i++) l[i] *= fac_s[r0 + i];
          }
          if (cnt > c0) {
            // O^T holds sums relative to the old references: wait for the tile before this one, then rescale this thread's part
            ok = wait(bar(bPdone + (cnt - 1) % kSB), ((cnt - 1) / kSB) & 1, 66, cnt UQ_PROF_SITE(0));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int db = 0; db < C::kDB; db++) {
              float ov[HW];
              load_scores(lane_addr + C::cO + db * NT + r0, ov);
#pragma unroll
              for (int i = 0; i < HW; i++) ov[i] *= facO_s[r0 + i];
              store_cols(lane_addr + C::cO + db * NT + r0, ov);
            }
          }
          mcur ^= 1;   // the next tile's rendezvous keeps fac / wmax / wr from being overwritten while still read
          load_masked();
          probabilities(mref + mcur * NT);
          write_p((int)wr[4 + mcur]);
        }
        UQ_PROF_TA2
        if (!((UQ_ABL & 16) && lean)) {
#pragma unroll
          for (int i = 0; i < HW; i += 2) add_f32x2(l[i], l[i + 1], pv[i], pv[i + 1]);
        }
        tc_fence_before();
        fence_async_smem();
        warp_arrive(bar(bPfull + buf));   // P^T is written; it also tells the Q.K issuer that this slot's S^T is consumed
        if (st == 0) { UQ_TRACE(13, cnt) }
        UQ_TRACE_CTA_T(3)
        if (cnt == 0) { UQ_TRACE_CTA_T(2) }
        UQ_PROF_TB(5)
      }
      if (!ok) break;
      UQ_TRACE_SEG(5)
      // ---- segment epilogue: row sums over the 128 keys, then O^T -> normalised partial
      {
        const float lw = warp_fold<HW, false>(l, lane);
        // one partial per warp (quarter of the keys) and row; the readers add the four in a fixed order, so that the result
        // does not depend on which warp got there first
        if ((lane & (32 / HW - 1)) == 0) lsum[quad * NT + r0 + warp_fold_row<HW>(lane)] = lw;
      }
      UQ_TRACE_SEG(6)
      ok = rendezvous(70, seg_i);
      UQ_TRACE_SEG(7)
      if (ok) ok = wait(bar(bOdone), seg_i & 1, 71, seg_i UQ_PROF_SITE(0));
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      UQ_TRACE_SEG(8)
      {
        const size_t slot = uq_slot(p, sg.b, sg.hk, sg.slot);
        float* mo = p.mo + slot * x.BM * D;
        float* ml = p.ml + slot * x.BM;
        const float* mr = mref + mcur * NT;
        const float osc = pow2_f32((int)wr[4 + mcur] - 127);   // O^T was accumulated relative to the segment's V reference
        bool bad = false;   // an infinity or a NaN in the sums: a probability or a V value overflowed fp16 somewhere in the segment
        // a warp's threads share their HW rows: lane i works out row r0 + i's factor osc / sum once (-1: the row saw nothing),
        // the stores fetch it by shuffle
        float f_mine = -1.f;
        if (lane < HW && r0 + lane < rows) {
          const int r = r0 + lane;
          const float lr = (lsum[r] + lsum[NT + r]) + (lsum[2 * NT + r] + lsum[3 * NT + r]);
          bad = !(lr <= 3.0e38f);
          if (lr > 0.f) f_mine = __fdividef(osc, lr);
        }
#pragma unroll
        for (int db = 0; db < C::kDB; db++) {
          float ov[HW];
          load_scores(lane_addr + C::cO + db * NT + r0, ov);   // accumulator lane kk of block db = channel 128 db + kk
#pragma unroll
          for (int i = 0; i < HW; i++) {
            const float f = __shfl_sync(0xffffffffu, f_mine, i);
            const int r = r0 + i;
            if (r < rows && db * 128 + kk < D) {                // head_dim 64: the upper 64 lanes are a copy
              bad |= !(fabsf(ov[i]) <= 3.0e38f);
              mo[(size_t)r * D + db * 128 + kk] = f >= 0.f ? ov[i] * f : 0.f;
            }
          }
        }
        // quick path: the segment's result is garbage then; the second pass computes it again on the careful path
        if (!UQ_ABL && !careful && __any_sync(0xffffffffu, bad) && lane == 0) { atomicOr(&redo[ord >> 5], 1u << (ord & 31)); redo[kRedoWords] = 1u; }
        if (st < rows) { const float lr = (lsum[st] + lsum[NT + st]) + (lsum[2 * NT + st] + lsum[3 * NT + st]); ml[st] = lr > 0.f ? mr[st] + log2f(lr) : -INFINITY; }
      }
      tc_fence_before();
      warp_arrive(bar(bEpi));
      UQ_TRACE_SEG(9)
      // (no rendezvous here: the next segment initialises the sums and references only after the rendezvous in the middle of
      // its prologue, which every thread reaches after it has read them above)
      seg_i++;
    }
    UQ_PROF_FLUSH(4, st == 0)
  }

  // ---- end of a pass: every role gets here (all waits are bounded)
  tc_fence_before();
  __syncthreads();
  if (*abort_flag || !*reinterpret_cast<volatile uint32_t*>(&redo[kRedoWords])) break;
  }
  UQ_TRACE_CTA_T(4)
  UQ_TRACE_CTA_V(5, cnt)
  UQ_TRACE_CTA_V(6, seg_i)
  // ---- common exit: TMEM goes back before the CTA ends
  if (warp == kWarpMma) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    else
      cudaGetLastError();
  }
  return fn;
}

// The code arrays as a 2-D byte tensor [cache rows][D/2]; a box is one page of one head (`page` rows: PAGE, or 128 for larger pages).  The number
// of physical pages is not part of the launch arguments, so the row extent is the largest the map can hold:
// only rows named by the page table are ever touched.
bool make_code_map(CUtensorMap* map, const uint8_t* base, int code_row_bytes, int page) {
  // the swizzle span equals the code row (32 / 64 / 128 bytes): a thread reading its key's row then hits every bank once
  const CUtensorMapSwizzle swz = code_row_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : (code_row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)code_row_bytes, (cuuint64_t)1 << 31};
  const cuuint64_t strides[1] = {(cuuint64_t)code_row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)code_row_bytes, (cuuint32_t)page};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The K codes for the block-scaled contraction: the same rows as packed 4-bit elements, which the copy engine unpacks on the
// way in (16 elements = 8 bytes, then 8 bytes of padding), so a key's 128 channels land as one 128-byte row, 128-byte swizzle.
bool make_unpack_map(CUtensorMap* map, const uint8_t* base, int channels, int page) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)channels, (cuuint64_t)1 << 31};
  const cuuint64_t strides[1] = {(cuuint64_t)channels / 2};
  const cuuint32_t box[2] = {(cuuint32_t)channels, (cuuint32_t)page};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<uint8_t*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The tensor maps of the caches this thread used last (a serving loop calls with the same few caches over and over: encoding
// a map costs the host a microsecond or two per call).  A map depends on the base address, the row width and the box only.
struct MapKey {
  const void* base;
  int row_bytes, box_rows, unpack;
  bool operator==(const MapKey& o) const { return base == o.base && row_bytes == o.row_bytes && box_rows == o.box_rows && unpack == o.unpack; }
};
bool cached_map(CUtensorMap* out, const MapKey& key) {
  constexpr int kSlots = 16;
  thread_local MapKey keys[kSlots] = {};
  thread_local CUtensorMap maps[kSlots];
  thread_local int used = 0, next = 0;
  for (int i = 0; i < used; i++)
    if (keys[i] == key) { *out = maps[i]; return true; }
  CUtensorMap m;
  const uint8_t* base = static_cast<const uint8_t*>(key.base);
  if (!(key.unpack ? make_unpack_map(&m, base, key.row_bytes * 2, key.box_rows) : make_code_map(&m, base, key.row_bytes, key.box_rows))) return false;
  const int slot = used < kSlots ? used++ : (next = (next + 1) % kSlots);
  keys[slot] = key;
  maps[slot] = m;
  *out = m;
  return true;
}

template <int D, int NT, int FMT>
cudaError_t launch(const UQParams& p, const UQLaunch& x, cudaStream_t s) {
  using C = Cfg<D, NT, FMT>;
  auto kern = uq_verify_tc_kernel<D, NT, FMT>;
  static std::atomic<bool> ready[64];
  static std::atomic<int> sm_counts[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!ready[dev].load(std::memory_order_acquire)) {   // per device: the attribute belongs to the device's copy of the kernel
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
    if (e != cudaSuccess) { cudaGetLastError(); return e; }
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    sm_counts[dev].store(n, std::memory_order_relaxed);
    ready[dev].store(true, std::memory_order_release);
  }
  Params prm;
  prm.p = p;
  prm.x = x;
  // an item of n tiles cut into chunks of c tiles spans at most ceil(n / c) + 1 CTAs: keep that within ns_eff
  const long long max_tiles = ((long long)p.max_pages * p.PAGE + kKeys - 1) / kKeys;
  prm.chunk_min = x.ns_eff >= 2 ? (int)((max_tiles + x.ns_eff - 2) / (x.ns_eff - 1)) : 1;
  CUtensorMap mk, mv;
  int box_rows = kKeys;   // a copy moves gcd(PAGE, 128) tokens: a page of up to 128 tokens, a 128-token part of a larger one, or their common part
  while (p.PAGE % box_rows) box_rows >>= 1;
  prm.unit = box_rows;
  if (!cached_map(&mk, MapKey{p.kc, C::kCodeRow, box_rows, C::kBS ? 1 : 0}) || !cached_map(&mv, MapKey{p.vc, C::kCodeRow, box_rows, 0})) return cudaErrorInvalidValue;
  const int sms = sm_counts[dev].load(std::memory_order_relaxed);
  if (sms <= 0) return cudaErrorInitializationError;
  kern<<<sms, cta_threads(NT), C::kSmem, s>>>(prm, mk, mv);
  return cudaGetLastError();
}

}  // namespace tc

#ifdef UQ_TC_TRACE
extern "C" int uqb_debug_tc_cta(unsigned long long* out1280) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out1280, tc::g_tc_cta, sizeof(unsigned long long) * 1280);
  return (int)e;
}
extern "C" int uqb_debug_tc_trace(long long* out1024) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out1024, tc::g_tc_trace, sizeof(long long) * 1024);
  return (int)e;
}
#endif
#ifdef UQ_TC_PROF
// profiling build only: read and clear the per-role cycle counters (5 roles x 8 counters)
extern "C" int uqb_debug_tc_prof(unsigned long long* out40) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out40, tc::g_tc_prof, sizeof(unsigned long long) * 40);
  static const unsigned long long zero[40] = {0};
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(tc::g_tc_prof, zero, sizeof(zero));
  return (int)e;
}
#endif

bool uq_verify_tc_serves(const UQParams& p, const UQLaunch& x) {
  if (p.fmt != 0 && p.fmt != 1) return false;
  if (!(p.D == 64 || p.D == 128 || p.D == 256)) return false;
  if (p.PAGE < 16 || p.PAGE > 1024 || p.PAGE % 16) return false;   // multiples of 16 tokens: copies of gcd(PAGE, 128) >= 16 tokens tile both the page and the 128-key tile
  if (x.rows > 64 || p.B > tc::Cfg<128, 64>::kMaxB) return false;
  if ((reinterpret_cast<uintptr_t>(p.kc) | reinterpret_cast<uintptr_t>(p.vc) | reinterpret_cast<uintptr_t>(p.ks) | reinterpret_cast<uintptr_t>(p.vs)) & 15) return false;
  if (p.fmt == 0 && tc::block_scaled(p.D) && (reinterpret_cast<uintptr_t>(p.kc) & 31)) return false;   // the unpacking tensor map wants 32-byte alignment
  if ((long long)p.max_pages * p.PAGE >= (1ll << 30)) return false;
  return tc::encode_fn() != nullptr;
}

// Partial slots the kernel uses per (sequence, kv head): at most the caller's nsplit, and no more than an item can span.
// The flat list gives a CTA ceil(total / SMs) tiles and total >= Hkv x (tiles of the longest item), so an item spans at
// most ceil(SMs / Hkv) + 1 CTAs; slots beyond that would only be marked empty by the kernel and skipped by the combine.
int uq_verify_tc_splits(const UQParams& p, const UQLaunch&) {
  static std::atomic<int> cached[64];
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64) sms = cached[dev].load(std::memory_order_relaxed);
  if (sms <= 0) {
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) { cudaGetLastError(); return p.nsplit; }
    if (dev >= 0 && dev < 64) cached[dev].store(sms, std::memory_order_relaxed);
  }
  const int span = (sms + p.HKV - 1) / p.HKV + 1;
  return std::max(1, std::min(p.nsplit, span));
}

template <int D, int FMT>
static cudaError_t dispatch_rows(const UQParams& p, const UQLaunch& x, cudaStream_t s) {
  if (x.rows <= 16) return tc::launch<D, 16, FMT>(p, x, s);
  if (x.rows <= 32) return tc::launch<D, 32, FMT>(p, x, s);
  return tc::launch<D, 64, FMT>(p, x, s);
}

cudaError_t uq_verify_tc_dispatch(const UQParams& p, const UQLaunch& x, cudaStream_t s) {
  switch (p.D) {
    case 64: return p.fmt == 1 ? dispatch_rows<64, 1>(p, x, s) : dispatch_rows<64, 0>(p, x, s);
    case 128: return p.fmt == 1 ? dispatch_rows<128, 1>(p, x, s) : dispatch_rows<128, 0>(p, x, s);
    case 256: return p.fmt == 1 ? dispatch_rows<256, 1>(p, x, s) : dispatch_rows<256, 0>(p, x, s);
  }
  return cudaErrorInvalidValue;
}
