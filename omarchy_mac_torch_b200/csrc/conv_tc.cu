// Tensor-core implicit-GEMM convolution for sm_100a: tcgen05.mma (kind::tf32) with the accumulator in TMEM, operands
// staged in shared memory by TMA (im2col-mode loads for the activation operand, tiled loads for the weights), and a
// 3xTF32 split so float32 accuracy holds:  a*b ~= a_lo*b_hi + a_hi*b_lo + a_hi*b_hi  with x_hi = tf32(x), x_lo = tf32(x - x_hi).
//
// GEMM view (forward): D[m, co] = sum_k A[m, k] * W[co, k],  m = (img, oy, ox),  k = (ky, kx, c) with c innermost in
// blocks of 32 floats (one 128-byte swizzle row). The activation must be channels-last with c % 4 == 0 so that a pixel's
// channel run starts on a 16-byte boundary (a TMA requirement). Weights are re-laid out per call into [2][co][ky][kx][c
// padded to 32] (hi and lo planes, zero padded) by a small kernel; they are tiny next to the activations.
//
// Persistent kernel: one CTA per SM walks 128 x BN output tiles. Warp roles (320 threads):
//   warp 0       TMA producer: per k-block one im2col load of A (128 pixels x 32 channels of one filter tap) and two tiled
//                loads of W (hi and lo planes), all completing on the stage's "loaded" mbarrier
//   warp 1       allocates TMEM; one lane issues the MMAs: per 8-wide k-step three tcgen05.mma, then tcgen05.commit to
//                free the stage; a final commit signals the epilogue
//   warps 2..5   produce A_lo next to the A tile TMA wrote (which serves as A_hi), arrive on the stage's "split" mbarrier
//   warps 10..13 epilogue: tcgen05.ld of their 32-lane quarter of the accumulators, bias / ReLU, store in the output's layout;
//                when TMEM holds two tiles' accumulators the epilogue of tile i overlaps the main loop of tile i+1
//   warps 6..9   join the split warps when the reduction is long, the epilogue warps when it is short
// Every mbarrier wait is bounded by a clock budget; on expiry the kernel raises an error word, all roles leave their loops,
// TMEM is freed and the kernel returns (the host reports it as a failed launch at the next synchronisation).
//
// The weight gradient is a second kernel with the same machinery and both operands "MN-major": D[co, (tap, c)] = sum over
// pixels of gy[pix, co] * im2col(x)[pix, (tap, c)]. The reduction runs over pixels, which is the row index of both
// channels-last operands, so each 32-pixel x 32-channel TMA box is one column of swizzle atoms of an MN-major UMMA operand.
// Pixels are split over blockIdx.z; partial tiles go to slabs that a second kernel sums in a fixed order (deterministic),
// re-laying [co][tap][c] out as [co][ci][ky][kx]. Both operands are activations, so both are split hi/lo in shared memory.
//
// The input gradient of a stride-1 convolution is the same kernel: a forward convolution of gy with the weights transposed
// and flipped (done by the weight re-layout kernel). Replaces the reference's generated kinds 0 and 1
// (omarchy_mac_torch/gemm.py:25-59) for the geometries it accepts; everything else stays on the exact-fp32 path.
#include <cuda.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <mutex>
#include <numeric>

#include "common.cuh"

namespace omt {

thread_local PlanOverride tl_plan{0, 0.0};

namespace {

constexpr int BM = 128;        // output pixels per tile (UMMA M)
constexpr int BKF = 32;        // floats per k-block (128 bytes)
constexpr int UMMA_K = 8;      // tf32 MMA depth
constexpr int TC_THREADS = 448;  // producer warp, MMA warp, 4 split warps, 8 epilogue warps
constexpr long long WAIT_BUDGET_CLOCKS = 2000000000ll;  // ~1 s at B200 clocks
constexpr int FLEX_SPLIT_KBLOCKS = 8;  // from this many k-blocks per tile on, warps 6..9 split operands instead of storing tiles
constexpr int BNSTATS_MIN_KBLOCKS = 16;            // epilogue statistics: from this reduction length on ...
constexpr int64_t BNSTATS_SMALL_OUTPUT = 32 << 20;  // ... or when the output has at most this many elements
constexpr int PAIR_MIN_KBLOCKS = 8;   // CTA pairs from this reduction length on (measured: +2..6 % from 8 k-blocks, -6..9 % at 2..4)
constexpr int ACC1_MAX_KBLOCKS = 36;  // single-accumulator 128 x 256 tiles up to K = 1152 (error below 1e-5 of the largest output)

__device__ int g_tc_error = 0;  // first failure: 1 = mbarrier wait expired

// ---------------------------------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// CLUSTER: acquire at cluster scope, for a barrier that threads of the other CTA of a pair arrive on
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  if constexpr (CLUSTER)
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the budget expired or another role already gave up.
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try<CLUSTER>(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; i++)
      if (mbar_try<CLUSTER>(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > WAIT_BUDGET_CLOCKS) {
      *abort_flag = 1;
      atomicCAS(&g_tc_error, 0, 1);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_im2col_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c, int w, int h, int n, uint16_t ow,
                                              uint16_t oh) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(ow), "h"(oh)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_im2col_4d(const CUtensorMap* map, int c, int w, int h, int n, uint16_t ow, uint16_t oh) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.im2col [%0, {%1, %2, %3, %4}], {%5, %6};" ::"l"(map), "r"(c), "r"(w), "r"(h), "r"(n),
               "h"(ow), "h"(oh)
               : "memory");
}
__device__ __forceinline__ void tma_tile_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ void tma_tile_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z, int w, int v) {
  asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w), "r"(v)
               : "memory");
}
__device__ __forceinline__ void tma_tile_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// ---- CTA pairs (cta_group::2): two CTAs of a cluster, on the two SMs of a TPC, run one MMA of 256 rows. Each holds its own 128
// rows of A and HALF of the B tile in shared memory, its own 128 x N accumulator in TMEM; CTA rank 0 issues for both. ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_count_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
// the shared::cluster address of `addr` (a shared::cta address of this CTA's layout) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {  // release at cluster scope: a barrier in either CTA of the pair
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {  // every thread of both CTAs
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// B tile rows of this CTA; the bytes are counted on the barrier `cluster_bar` of CTA rank 0
__device__ __forceinline__ void tma_tile_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at this offset in BOTH CTAs of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)3)
               : "memory");
}
// A operand from tensor memory (lane = row, one column per tf32 element), B from shared memory
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the calling warp's 32 lanes x 16 columns from registers: lane i writes v[0..15] to columns [col, col + 16) of its TMEM lane
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// two 32-column loads (same lanes, two column ranges) and the wait, as one statement so that no use of the registers can be
// scheduled before the wait
__device__ __forceinline__ void tmem_ld32x2(uint32_t ta, uint32_t tb, uint32_t (&a)[32], uint32_t (&b)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]), "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]), "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31]),
        "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]), "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]), "=r"(b[16]), "=r"(b[17]), "=r"(b[18]), "=r"(b[19]), "=r"(b[20]), "=r"(b[21]), "=r"(b[22]), "=r"(b[23]), "=r"(b[24]), "=r"(b[25]), "=r"(b[26]), "=r"(b[27]), "=r"(b[28]), "=r"(b[29]), "=r"(b[30]), "=r"(b[31])
      : "r"(ta), "r"(tb)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t ta, uint32_t (&a)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]), "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]), "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31])
      : "r"(ta)
      : "memory");
}
__device__ __forceinline__ float tf32_rna(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}
// 3xTF32 operand split. The tensor core reads a tf32 operand as the top 19 bits of the fp32 word in shared memory (the low
// 13 mantissa bits are ignored), so the buffer TMA wrote already is the "hi" operand: hi = x with those bits cleared. Only
// lo = x - hi (exact in fp32, then rounded to tf32) has to be produced, which saves one of the two shared-memory stores.
#ifndef OMT_TC_IMPLICIT_HI
#define OMT_TC_IMPLICIT_HI 1
#endif
__device__ __forceinline__ uint4 split_lo(uint4 v, uint4& h) {
  float f0 = __uint_as_float(v.x), f1 = __uint_as_float(v.y), f2 = __uint_as_float(v.z), f3 = __uint_as_float(v.w);
#if OMT_TC_IMPLICIT_HI
  h.x = v.x & 0xffffe000u; h.y = v.y & 0xffffe000u; h.z = v.z & 0xffffe000u; h.w = v.w & 0xffffe000u;
#else
  h.x = __float_as_uint(tf32_rna(f0)); h.y = __float_as_uint(tf32_rna(f1)); h.z = __float_as_uint(tf32_rna(f2)); h.w = __float_as_uint(tf32_rna(f3));
#endif
  uint4 l;
  l.x = __float_as_uint(tf32_rna(f0 - __uint_as_float(h.x))); l.y = __float_as_uint(tf32_rna(f1 - __uint_as_float(h.y)));
  l.z = __float_as_uint(tf32_rna(f2 - __uint_as_float(h.z))); l.w = __float_as_uint(tf32_rna(f3 - __uint_as_float(h.w)));
  return l;
}

// K-major operand tile with 128-byte rows and the 128B swizzle: 8-row atoms of 1024 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset: next 8-row atom
  d |= (uint64_t)1 << 46;                        // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}
constexpr uint32_t idesc_tf32(int n, bool mn_major = false, int m = BM) {  // m = 256: the rows of both CTAs of a pair
  return (1u << 4) /* D = f32 */ | (2u << 7) /* A = tf32 */ | (2u << 10) /* B = tf32 */ | (mn_major ? (3u << 15) : 0u) /* A, B majors */ |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// MN-major tf32 operand. The only shared-memory layout the tensor core accepts for it is "128B swizzle with 32-byte
// atomicity": 128-byte rows (32 floats along M/N) for consecutive k, 32-byte granules XOR-ed with the row index modulo 4, so
// the swizzle atom is 4 k-rows x 128 bytes. `chunk_bytes` separates consecutive 32-float runs along M/N (leading byte
// offset); groups of 4 k-rows follow each other every 512 bytes (stride byte offset). TMA writes this layout with
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t chunk_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(chunk_bytes >> 4) << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)1 << 61;  // SWIZZLE_128B_BASE32B
  return d;
}
__device__ __forceinline__ void tma_tile_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z),
               "r"(w)
               : "memory");
}

struct TcArgs {
  ActView y;          // output activation (any strides)
  const float* bias;
  // OMT_EPI_BNSTATS: per 32-row group g = 4 * (row tile) + (lane quarter) and channel the sum of the stored values and their
  // squared deviations from the group's own mean, stats[(2g + {0,1}) * N + channel], then the groups' row counts at
  // stats[2 * groups * N + g], then ceil(N / 32) zeroed words (ticket counters of the merging kernel). The merge
  // (bn_partials_kernel) runs in a fixed order: deterministic, and exact for any mean.
  float* stats;
  int M, N;           // GEMM extents: pixels, output channels
  int oh, ow;         // pixel grid of the GEMM rows (to decompose m)
  int low_h, low_w;   // input coordinate of tap (0,0) for output pixel (0,0): -pad for a forward convolution
  int cblocks;        // 32-channel blocks per tap
  uint32_t flags;
  int16_t kh, kw;     // filter taps of this (sub-)convolution
  int8_t stride;      // traversal stride over the input
  int8_t out_step, out_y0, out_x0;  // GEMM row (oy, ox) is stored at (oy*out_step + out_y0, ox*out_step + out_x0)
  int store_mode;     // 0: plain stores (any strides); 1: TMA stores of 32-row boxes of the [M, N] matrix; 2: of window rectangles
  int reserved_[3];   // keeps the struct at 128 bytes (see below)
  // The last 16 bytes are shared by two modes that never occur together (growing this struct by 16 bytes made every
  // tile of the kernel 2-3 us slower on the GPU, measured; the cause was not established, so its size is kept).
  //  * "window" mode (win_w != 0; few input channels): the A operand comes from a zero-padded [n][h][w][4] copy of the
  //    input through a tiled tensor map whose pixel dimension overlaps (stride = conv stride * 16 bytes), so one 32-float
  //    row holds 8 consecutive input pixels x 4 channels = the (kx, c) run of a filter row. GEMM rows are win_w x win_h
  //    pixel rectangles.
  //  * split-K (the SPLITK kernel instantiation only; win_w is not looked at there): for problems with fewer tiles than
  //    SMs, tile t = (output tile, split); a CTA reduces the k-blocks of its split and stores the raw sums to
  //    part[split][M][N]; splitk_epilogue_kernel adds the splits in order and applies the epilogue.
  union {
    struct { int win_w, win_h, tiles_x, tiles_y; };
    struct { int splits, unused_; float* part; };
  };
};
static_assert(sizeof(TcArgs) == 128, "TcArgs is a kernel parameter whose size is performance-sensitive");

// ACC1: one accumulator per tile instead of the (main, cross-term) pair. The main sum is then truncated three times per
// k-step instead of once, which costs accuracy in proportion to the reduction length (measured 1.6e-5 of the largest output at
// K = 2304 against 5.7e-6), so it is used only for 128 x 256 tiles with short reductions: there the pair fills TMEM, the
// epilogue cannot overlap the next tile's main loop, and with a short main loop that exposed epilogue is a large share.
// PAIR: the CTA is one of a cta_group::2 pair and stages only its half of the B tile (BN / 2 weight rows), which leaves room
// for a third stage at BN = 256.
// ATMEM (64-column tiles): the lo half of the A operand reaches the tensor core from tensor memory. The accumulators of the two
// tiles in flight take 256 of the 512 columns; the other 256 hold one 32-column A_lo tile per stage. Without A_lo a stage is
// 32 KB of shared memory, so the ring is six stages deep instead of four.
template <int BN, bool ACC1 = false, bool PAIR = false, bool ATMEM = false>
struct Smem {
  static constexpr int A_RING_COL = 256, A_STAGE_COLS = 32;
  static constexpr int STAGES = ATMEM ? 6 : (PAIR ? (BN == 256 ? 3 : 4) : (BN == 256 ? 2 : (BN == 128 ? 3 : 4)));
  static constexpr int ACC_COLS = ACC1 ? BN : 2 * BN;          // TMEM columns of one tile's accumulator(s)
  static constexpr int ACC_BUFS = ACC_COLS == 512 ? 1 : 2;     // tiles in flight in TMEM (512 columns in total at most)
  static constexpr int TMEM_COLS = ATMEM ? 512 : ACC_BUFS * ACC_COLS;  // 256 or 512: a power of two
  static constexpr int A_BYTES = BM * 128, B_BYTES = (PAIR ? BN / 2 : BN) * 128;
  static constexpr int B_OFF = ATMEM ? A_BYTES : 2 * A_BYTES;  // B_hi behind A_hi (and A_lo, when that lives in shared memory)
  static constexpr int STAGE_BYTES = B_OFF + 2 * B_BYTES;
  static constexpr int EPI_OFF = STAGES * STAGE_BYTES;          // per epilogue warp one 32-row x 128-byte store buffer
  static constexpr int EPI_BYTES = 8 * 4096;
  static constexpr int BAR_OFF = EPI_OFF + EPI_BYTES;
  static constexpr int NBARS = 3 * STAGES + 2 * ACC_BUFS + (PAIR ? STAGES : 0);  // a pair has separate "A loaded" / "B loaded" barriers
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;  // barriers + alignment slack
};

// ---------------------------------------------------------------------------------------------------------------------
// the kernel: persistent, one CTA per SM walking output tiles t = blockIdx.x, blockIdx.x + gridDim.x, ...
// ---------------------------------------------------------------------------------------------------------------------
struct TileCoord {
  int img0, oy0, ox0;  // first pixel of the tile (im2col mode: linear pixel run; window mode: top-left of the rectangle)
  int m0, n0;
};
__device__ __forceinline__ TileCoord decode_tile(const TcArgs& g, int t, int n_tiles, int bn, int splits, int win_w) {
  TileCoord c;
  t /= splits;
  const int mt = t / n_tiles;
  c.n0 = (t - mt * n_tiles) * bn;
  c.m0 = mt * BM;
  if (win_w) {
    const int per = g.tiles_x * g.tiles_y;
    c.img0 = mt / per;
    const int r = mt - c.img0 * per;
    c.oy0 = (r / g.tiles_x) * g.win_h; c.ox0 = (r % g.tiles_x) * win_w;
  } else {
    const int ohw = g.oh * g.ow;
    c.img0 = c.m0 / ohw;
    const int r0 = c.m0 - c.img0 * ohw;
    c.oy0 = r0 / g.ow; c.ox0 = r0 - c.oy0 * g.ow;
  }
  return c;
}

// PAIR (launched as clusters of two CTAs; the host picks it for an even number of row tiles): the pair works on row tiles 2p
// and 2p + 1 of the same 256 columns with ONE stream of tcgen05.mma.cta_group::2 instructions (M = 256) that CTA rank 0
// issues. Each CTA loads and splits its own A rows and loads half of the B tile, so per k-block a CTA moves 176 KB through
// shared memory instead of 256 KB -- the shared-memory bandwidth, not the tensor pipe, bounds the single-CTA kernel. Who
// signals what:
//   A loaded [s]   own CTA, by its TMA                        -> own split warps
//   B loaded [s]   rank 0's barrier, by both CTAs' TMA        -> rank 0's MMA thread
//   split    [s]   rank 0's barrier, split warps of both CTAs -> rank 0's MMA thread (also covers "A loaded" of both CTAs)
//   free     [s]   both CTAs (multicast commit)               -> own producer
//   acc full [b]   both CTAs (multicast commit)               -> own epilogue warps
//   acc empty[b]   rank 0's barrier, epilogue warps of both   -> rank 0's MMA thread
// ATMEM (64-column tiles): the split warps read the A tile once (each lane its own row) and put lo = tf32(x - hi) into tensor
// memory with tcgen05.st instead of into shared memory; the cross-term MMA takes its A operand from there (tcgen05.mma with a
// tensor-memory A). A stage then is A_hi + B in shared memory (32 KB), and the ring is six deep instead of four: these
// tiles wait for operands, not for the tensor pipe or shared memory (measured: 36 % tensor-active, 42 % of the L1 peak).
template <int BN, bool SPLITK, bool ACC1 = false, bool PAIR = false, bool ATMEM = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_y,
               const TcArgs g) {
  static_assert(!PAIR || !SPLITK, "CTA pairs: unsplit reduction");
  static_assert(!ATMEM || (BN == 64 && !SPLITK && !PAIR && !ACC1), "A from tensor memory: 64-column tiles");
  using S = Smem<BN, ACC1, PAIR, ATMEM>;
  static_assert(!ATMEM || S::STAGES * S::A_STAGE_COLS <= 512 - S::A_RING_COL, "the A ring must fit beside the accumulators");
  // k-blocks per barrier hand-off. A narrow tile's k-block is a few hundred tensor clocks, and the load -> split -> MMA -> free
  // chain costs about as much again in wake-ups, so the 64-column tiles move two k-blocks per hand-off: the ring of S::STAGES
  // k-block buffers is then RING groups of KPS, with one set of barriers per group.
  constexpr int KPS = ATMEM ? 2 : 1, RING = S::STAGES / KPS;
  static_assert(S::STAGES % KPS == 0, "whole groups");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
  // barrier indices: [0,S) loaded, [S,2S) split, [2S,3S) free, then ACC_BUFS x "accumulator full", ACC_BUFS x "accumulator drained"
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  constexpr int ACC_FULL = 3 * S::STAGES, ACC_EMPTY = 3 * S::STAGES + S::ACC_BUFS;
  constexpr int B_LOADED = 3 * S::STAGES + 2 * S::ACC_BUFS;  // PAIR only; BAR(s) is then "A loaded"
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  // a barrier of CTA rank 0 as both CTAs of a pair address it
  auto LEADER = [&](int i) { return PAIR ? mapa_rank(BAR(i), 0u) : BAR(i); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + S::NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + S::NBARS + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = g.kh * g.kw * g.cblocks;
  const int n_tiles = (g.N + BN - 1) / BN;
#ifdef OMT_TC_EXPERIMENTS  // timing experiments only (results are wrong with most of these): which role bounds a tile
  const int dbg = g.reserved_[0];  // 1 no stores, 2 no wait for the staging buffer, 4 no operand split, 8 no MMAs, 16 L2 prefetch, 32 no TMEM loads
#else
  constexpr int dbg = 0;
#endif
  int splits = 1;  // a compile-time 1 in the common instantiation
  if constexpr (SPLITK) splits = g.splits;
  const int win_w = SPLITK ? 0 : g.win_w;  // the split-K fields alias the window fields
  // GEMM row tiles: 128-pixel runs, or in window mode the rectangles of every image (M = images x oh x ow there)
  const int m_tiles = win_w ? (g.M / (g.oh * g.ow)) * g.tiles_x * g.tiles_y : (g.M + BM - 1) / BM;
  const int total_tiles = m_tiles * n_tiles * splits;
  // the CTA's (or the pair's) walk over the tiles: work item i of `work_items`, `work_step` apart, is this CTA's tile tile_of(i)
  const int work_items = PAIR ? (m_tiles / 2) * n_tiles : total_tiles;
  const int work_first = PAIR ? (int)cluster_id_x() : (int)blockIdx.x, work_step = PAIR ? (int)cluster_count_x() : (int)gridDim.x;
  auto tile_of = [n_tiles, rank](int i) -> int {
    if constexpr (!PAIR) return i;
    const int mp = i / n_tiles;
    return (2 * mp + (int)rank) * n_tiles + (i - mp * n_tiles);
  };
  // k-block range of split sp: [sp * kblocks / splits, (sp + 1) * kblocks / splits)
  auto kb_begin = [kblocks, splits](int t) -> int {
    if constexpr (!SPLITK) return 0;
    return (int)(((int64_t)(t % splits) * kblocks) / splits);
  };
  auto kb_end = [kblocks, splits](int t) -> int {
    if constexpr (!SPLITK) return kblocks;
    return (int)(((int64_t)(t % splits + 1) * kblocks) / splits);
  };

  // Warps 6..9 take the role that is short of hands: with a long reduction the tile's time goes to the main loop, where the
  // operand split sits between a stage's arrival and its MMAs, so they split (8 split warps, 4 epilogue warps); with a short
  // one the tile's time goes to storing it, so they run the epilogue (4 split warps, 8 epilogue warps).
  const int split_warps = kblocks / splits >= FLEX_SPLIT_KBLOCKS ? 8 : 4;
  if (threadIdx.x == 0) {
    constexpr int ctas = PAIR ? 2 : 1;  // arrivals from both CTAs meet on rank 0's barriers
    for (int s = 0; s < S::STAGES; s++) {
      mbar_init(BAR(s), 1);                    // loaded: one arrive.expect_tx + TMA bytes
      mbar_init(BAR(S::STAGES + s), ctas * split_warps);  // split: one arrival per split warp
      mbar_init(BAR(2 * S::STAGES + s), 1);    // free: tcgen05.commit
      if constexpr (PAIR) mbar_init(BAR(B_LOADED + s), 1);
    }
    for (int b = 0; b < S::ACC_BUFS; b++) {
      mbar_init(BAR(ACC_FULL + b), 1);         // tcgen05.commit after the tile's last MMA
      mbar_init(BAR(ACC_EMPTY + b), ctas * (12 - split_warps));  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // TMEM: per buffer two accumulators of BN fp32 columns (main sum, cross terms)
    if constexpr (PAIR) {  // the same warp of both CTAs, the same columns in both
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                   "r"((uint32_t)S::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                   "r"((uint32_t)S::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // the other CTA's barriers are initialised before anything here signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int i = work_first; i < work_items && ok; i += work_step) {
        const int t = tile_of(i);
        const TileCoord c = decode_tile(g, t, n_tiles, BN, splits, win_w);
        const int w0 = c.ox0 * g.stride + g.low_w, h0 = c.oy0 * g.stride + g.low_h;
        for (int kb = kb_begin(t), kbe = kb_end(t); kb < kbe; kb += KPS, it++) {
          const int s = it % RING, round = it / RING;
          if (round > 0 && !mbar_wait(BAR(2 * S::STAGES + s), (round - 1) & 1, abort_flag)) { ok = false; break; }
          if constexpr (KPS > 1) {  // a group of up to KPS k-blocks behind one "loaded" barrier
            const int nk = min(KPS, kbe - kb);
            mbar_expect_tx(BAR(s), nk * (S::A_BYTES + 2 * S::B_BYTES));
            for (int j = 0; j < nk; j++) {
              const int tap = (kb + j) / g.cblocks, cb = (kb + j) - tap * g.cblocks;
              const int ky = tap / g.kw, kx = tap - ky * g.kw;
              const uint32_t stage = smem_base + (s * KPS + j) * S::STAGE_BYTES;
              if (win_w) tma_tile_4d(stage, &map_a, BAR(s), cb * BKF, c.ox0, h0 + ky, c.img0);
              else tma_im2col_4d(stage, &map_a, BAR(s), cb * BKF, w0, h0, c.img0, (uint16_t)kx, (uint16_t)ky);
              tma_tile_3d(stage + S::B_OFF, &map_w, BAR(s), (tap * g.cblocks + cb) * BKF, c.n0, 0);
              tma_tile_3d(stage + S::B_OFF + S::B_BYTES, &map_w, BAR(s), (tap * g.cblocks + cb) * BKF, c.n0, 1);
            }
            continue;
          }
          const int tap = kb / g.cblocks, cb = kb - tap * g.cblocks;
          const int ky = tap / g.kw, kx = tap - ky * g.kw;
          const uint32_t stage = smem_base + s * S::STAGE_BYTES;
          if constexpr (PAIR) {
            // rank 0 announces the B bytes of both CTAs; the other CTA's copies may land first (the count goes negative until then)
            if (rank == 0) mbar_expect_tx(BAR(B_LOADED + s), 4 * S::B_BYTES);
            mbar_expect_tx(BAR(s), S::A_BYTES);
            tma_im2col_4d(stage, &map_a, BAR(s), cb * BKF, w0, h0, c.img0, (uint16_t)kx, (uint16_t)ky);
            const uint32_t bbar = LEADER(B_LOADED + s);
            const int row0 = c.n0 + (int)rank * (BN / 2);  // this CTA's half of the weight rows
            tma_tile_3d_pair(stage + S::B_OFF, &map_w, bbar, (tap * g.cblocks + cb) * BKF, row0, 0);
            tma_tile_3d_pair(stage + S::B_OFF + S::B_BYTES, &map_w, bbar, (tap * g.cblocks + cb) * BKF, row0, 1);
            continue;
          }
          mbar_expect_tx(BAR(s), S::A_BYTES + 2 * S::B_BYTES);
          if (win_w) tma_tile_4d(stage, &map_a, BAR(s), cb * BKF, c.ox0, h0 + ky, c.img0);  // kw == 1: tap = filter row
          else tma_im2col_4d(stage, &map_a, BAR(s), cb * BKF, w0, h0, c.img0, (uint16_t)kx, (uint16_t)ky);
          tma_tile_3d(stage + S::B_OFF, &map_w, BAR(s), (tap * g.cblocks + cb) * BKF, c.n0, 0);
          tma_tile_3d(stage + S::B_OFF + S::B_BYTES, &map_w, BAR(s), (tap * g.cblocks + cb) * BKF, c.n0, 1);
          if ((dbg & 16) && !win_w && t + (int)gridDim.x < total_tiles) {  // the same k-block of this CTA's next tile, into L2
            const TileCoord cn = decode_tile(g, t + gridDim.x, n_tiles, BN, splits, win_w);
            tma_prefetch_im2col_4d(&map_a, cb * BKF, cn.ox0 * g.stride + g.low_w, cn.oy0 * g.stride + g.low_h, cn.img0, (uint16_t)kx, (uint16_t)ky);
          }
        }
      }
      if (*abort_flag) {  // drain: let the copies already in flight land before the CTA exits (bounded)
        for (int k = max(0, it - RING); k < it; k++) {
          const long long t0 = clock64();
          while (!mbar_try(BAR(k % RING), (k / RING) & 1) && clock64() - t0 < WAIT_BUDGET_CLOCKS) {}
        }
      } else if (PAIR) {
        // the last stages' "free" arrivals come from the other SM's commit: let them land in this CTA's barriers before it exits
        for (int k = max(0, it - RING); k < it; k++)
          if (!mbar_wait(BAR(2 * S::STAGES + k % RING), (k / RING) & 1, abort_flag)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && rank == 0) {  // (of a pair, only CTA rank 0 issues: its instructions drive both SMs' tensor cores)
      constexpr uint32_t idesc = idesc_tf32(BN, false, PAIR ? 2 * BM : BM);
      // one instruction stream for both forms: `mma` multiplies 128 (or, for a pair, 256) rows of A by the BN columns of B
      auto mma = [](uint32_t d, uint64_t da, uint64_t db, uint32_t id, uint32_t accumulate) {
        if constexpr (PAIR) umma_tf32_pair(d, da, db, id, accumulate);
        else umma_tf32(d, da, db, id, accumulate);
      };
      auto commit = [](uint32_t bar) {
        if constexpr (PAIR) umma_commit_pair(bar);
        else umma_commit(bar);
      };
      int it = 0, tl = 0;
      bool ok = true;
      for (int i = work_first; i < work_items && ok; i += work_step, tl++) {
        const int t = tile_of(i);
        const int b = tl % S::ACC_BUFS, use = tl / S::ACC_BUFS;
        if (use > 0) {  // the epilogue must have drained this accumulator pair
          ok = mbar_wait<PAIR>(BAR(ACC_EMPTY + b), (use - 1) & 1, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t acc = tmem_base + b * S::ACC_COLS;
        const uint32_t cross = ACC1 ? acc : acc + BN;  // where the 2^-11-sized cross terms accumulate
        const int kb0 = kb_begin(t);
        for (int kb = kb0, kbe = kb_end(t); kb < kbe; kb += KPS, it++) {
          const int s = it % RING, round = it / RING;
          // One CTA: the products that need only what TMA loaded (a_hi x b_hi, a_hi x b_lo) are issued as soon as the stage has
          // landed, while the split warps still produce a_lo; the a_lo x b_hi products follow when "split" arrives. That takes the
          // split out of the load -> split -> MMA -> free chain for two thirds of the tensor work.
          // (For a pair "split" also stands for "A loaded" in both CTAs, so everything waits for it there.)
          auto split_done = [&]() {
            const bool r = mbar_wait<PAIR>(BAR(S::STAGES + s), round & 1, abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            return r;
          };
          // (The 64-column tiles with two k-blocks per hand-off measured slower that way -- 0.430 against 0.403 ms on 64 -> 64
          // 3x3 -- and wait for the split first, like the pairs.)
          ok = (!(PAIR || KPS > 1) || split_done()) && mbar_wait(BAR(PAIR ? B_LOADED + s : s), round & 1, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if constexpr (KPS > 1) {  // (ATMEM) the group's k-blocks one after the other, one commit
            constexpr uint32_t idesc_wide = idesc_tf32(2 * BN);
            const int nk = min(KPS, kbe - kb);
            for (int j = 0; j < nk; j++) {
              const int ss = s * KPS + j;
              const uint32_t stage = smem_base + ss * S::STAGE_BYTES;
              const uint64_t a_hi = smem_desc_sw128(stage), b_hi = smem_desc_sw128(stage + S::B_OFF);
#pragma unroll
              for (int k = 0; k < BKF / UMMA_K; k++) {
                const uint64_t adv = (uint64_t)((k * UMMA_K * 4) >> 4);
                umma_tf32(acc, a_hi + adv, b_hi + adv, idesc_wide, ((kb + j - kb0) | k) ? 1u : 0u);  // A_hi is the tile TMA wrote: from shared memory
                umma_tf32_ts(cross, tmem_base + S::A_RING_COL + ss * S::A_STAGE_COLS + k * UMMA_K, b_hi + adv, idesc, 1u);
              }
            }
            commit(BAR(2 * S::STAGES + s));
            continue;
          }
          const uint32_t stage = smem_base + s * S::STAGE_BYTES;
          const uint64_t a_hi = smem_desc_sw128(stage), a_lo = smem_desc_sw128(stage + S::A_BYTES);
          const uint64_t b_hi = smem_desc_sw128(stage + S::B_OFF), b_lo = smem_desc_sw128(stage + S::B_OFF + S::B_BYTES);
          if constexpr (!PAIR) {
#pragma unroll
            for (int k = 0; k < BKF / UMMA_K; k++) {
              if (dbg & 8) break;
              const uint64_t adv = (uint64_t)((k * UMMA_K * 4) >> 4);
              const uint32_t accumulate = ((kb - kb0) | k) ? 1u : 0u;  // the split's first MMA overwrites the accumulators
              if constexpr (!ACC1 && 2 * BN <= 256) {
                // B_lo follows B_hi in the stage, and the cross-term accumulator follows the main one in TMEM: one MMA of width
                // 2*BN over [B_hi; B_lo] yields a_hi*b_hi and a_hi*b_lo at once
                umma_tf32(acc, a_hi + adv, b_hi + adv, idesc_tf32(2 * BN), accumulate);
              } else {
                umma_tf32(acc, a_hi + adv, b_hi + adv, idesc, accumulate);
                umma_tf32(cross, a_hi + adv, b_lo + adv, idesc, ACC1 ? 1u : accumulate);
              }
            }
            ok = split_done();
            if (!ok) break;
#pragma unroll
            for (int k = 0; k < BKF / UMMA_K; k++) {
              if (dbg & 8) break;
              umma_tf32(cross, a_lo + (uint64_t)((k * UMMA_K * 4) >> 4), b_hi + (uint64_t)((k * UMMA_K * 4) >> 4), idesc, 1u);
            }
            commit(BAR(2 * S::STAGES + s));
            continue;
          }
#pragma unroll
          for (int k = 0; k < BKF / UMMA_K; k++) {
            if (dbg & 8) break;
            const uint64_t adv = (uint64_t)((k * UMMA_K * 4) >> 4);  // 32 bytes per k-step inside the swizzled row
            // two accumulators: the cross terms (2^-11 of the result) go to columns [BN, 2BN) so that the truncation the
            // tensor core applies on every accumulate hits the main sum once per k-step instead of three times
            const uint32_t accumulate = ((kb - kb0) | k) ? 1u : 0u;  // the split's first MMA overwrites the accumulators
            if constexpr (!ACC1 && !PAIR && 2 * BN <= 256) {
              // B_lo follows B_hi in the stage, and the cross-term accumulator follows the main one in TMEM: one MMA of width
              // 2*BN over [B_hi; B_lo] yields a_hi*b_hi and a_hi*b_lo at once, reading A_hi from shared memory once instead of
              // twice (these narrow tiles are bound by operand reads from shared memory, not by the tensor pipe)
              constexpr uint32_t idesc_wide = idesc_tf32(2 * BN);
              umma_tf32(acc, a_hi + adv, b_hi + adv, idesc_wide, accumulate);
              umma_tf32(cross, a_lo + adv, b_hi + adv, idesc, 1u);
            } else {
              mma(cross, a_lo + adv, b_hi + adv, idesc, accumulate);
              mma(cross, a_hi + adv, b_lo + adv, idesc, 1u);
              mma(acc, a_hi + adv, b_hi + adv, idesc, ACC1 ? 1u : accumulate);
            }
          }
          commit(BAR(2 * S::STAGES + s));  // stage is free once these MMAs have read it
        }
        if (ok) commit(BAR(ACC_FULL + b));  // this tile's accumulators are complete
      }
    }
  } else if (warp < 2 + split_warps) {
    // ---------------- operand split (warps 2..5, or 2..9) ----------------
    const int t4 = threadIdx.x - 64, split_threads = split_warps * 32;  // 0..127 or 0..255
    int it = 0;
    bool ok = true;
    for (int i = work_first; i < work_items && ok; i += work_step) {
      const int t = tile_of(i);
      for (int kb = kb_begin(t), kbe = kb_end(t); kb < kbe; kb += KPS, it++) {
        const int s = it % RING, round = it / RING;
        ok = mbar_wait(BAR(s), round & 1, abort_flag);
        if (!ok) break;
        if constexpr (ATMEM) {
          // lane = row of the tile's lane quarter this warp may touch in tensor memory; with eight split warps two share a
          // quarter and take 16 of the 32 k-columns each. A row is 128 bytes, its 16-byte chunks XOR-swizzled by (row & 7).
          const int q = warp & 3, halves = split_warps / 4, half = halves == 1 ? 0 : (warp - 2) >> 2;
          const int row = q * 32 + lane;
          const int nk = min(KPS, kbe - kb);
          for (int jb = 0; jb < nk; jb++) {
            const int ss = s * KPS + jb;
            const uint8_t* rp = smem + ss * S::STAGE_BYTES + row * 128;
            const uint32_t tcol = tmem_base + ((uint32_t)(q * 32) << 16) + S::A_RING_COL + ss * S::A_STAGE_COLS;
            for (int c16 = half; c16 < 2; c16 += halves) {  // columns [16 * c16, 16 * c16 + 16)
              uint32_t l[16];
#pragma unroll
              for (int j = 0; j < 4; j++) {
                const uint4 v = *reinterpret_cast<const uint4*>(rp + (((c16 * 4 + j) ^ (row & 7)) << 4));
                uint4 hh;
                const uint4 ll = split_lo(v, hh);
                l[4 * j] = ll.x; l[4 * j + 1] = ll.y; l[4 * j + 2] = ll.z; l[4 * j + 3] = ll.w;
              }
              tmem_st16(tcol + 16 * c16, l);
            }
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR(S::STAGES + s));
          continue;
        }
        uint4* hi = reinterpret_cast<uint4*>(smem + s * S::STAGE_BYTES);
        uint4* lo = reinterpret_cast<uint4*>(smem + s * S::STAGE_BYTES + S::A_BYTES);
#pragma unroll 4
        for (int idx = t4; idx < S::A_BYTES / 16; idx += split_threads) {
          if (dbg & 4) break;
          uint4 h;
          const uint4 l = split_lo(hi[idx], h);
#if !OMT_TC_IMPLICIT_HI
          hi[idx] = h;
#endif
          lo[idx] = l;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster(LEADER(S::STAGES + s));
          else mbar_arrive(BAR(S::STAGES + s));
        }
      }
    }
  } else {
    // ---------------- epilogue (warps 6..13, or 10..13): overlaps the next tile's main loop when ACC_BUFS == 2 ----------------
    // Two warps per TMEM lane quarter, each taking every other 32-column chunk, or one taking them all.
    const int q = warp & 3;           // TMEM lane quarter this warp may read
    const int halves = split_warps == 8 ? 1 : 2;        // epilogue warps per lane quarter
    const int half = halves == 1 ? 0 : (warp - 6) >> 2;
    // Dense channels-last outputs leave through shared memory: the warp lays its 32 rows x 32 channels out with the 128-byte
    // swizzle (conflict-free 16-byte stores) and one lane issues a TMA store of the box, which clips rows and channels that
    // fall outside the tensor.
    uint8_t* buf = smem + S::EPI_OFF + (warp - 6) * 4096;
    int tl = 0;
    bool ok = true;
    for (int i = work_first; i < work_items && ok; i += work_step, tl++) {
      const int t = tile_of(i);
      const int b = tl % S::ACC_BUFS, use = tl / S::ACC_BUFS;
      ok = mbar_wait(BAR(ACC_FULL + b), use & 1, abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const TileCoord c = decode_tile(g, t, n_tiles, BN, splits, win_w);
      const uint32_t acc = tmem_base + b * S::ACC_COLS + ((uint32_t)(q * 32) << 16);
      const int r = q * 32 + lane;
      int img, oy, ox;
      bool valid;
      if (win_w) {
        img = c.img0; oy = c.oy0 + r / win_w; ox = c.ox0 + r % win_w;
        valid = oy < g.oh && ox < g.ow;
      } else {
        const int m = c.m0 + r, ohw = g.oh * g.ow;
        valid = m < g.M;
        img = m / ohw;
        const int rr = m - img * ohw;
        oy = rr / g.ow; ox = rr - oy * g.ow;
      }
      if (!valid) { img = 0; oy = 0; ox = 0; }
      float* yrow = g.y.p + g.y.off(img, 0, oy * g.out_step + g.out_y0, ox * g.out_step + g.out_x0);
      const bool vec = g.y.sc == 1 && ((reinterpret_cast<uintptr_t>(yrow) & 15) == 0);
#pragma unroll 1
      for (int ch = half; ch < BN / 32; ch += halves) {
        uint32_t v[32], u[32];
        if (dbg & 32) {
#pragma unroll
          for (int j = 0; j < 32; j++) { v[j] = 0u; u[j] = 0u; }
        } else if constexpr (ACC1) {
          tmem_ld32(acc + ch * 32, v);
#pragma unroll
          for (int j = 0; j < 32; j++) u[j] = 0u;  // +0.f below: folded away
        } else {
          tmem_ld32x2(acc + ch * 32, acc + BN + ch * 32, v, u);
        }
        const int nb = c.n0 + ch * 32;
        if (nb >= g.N) continue;
        if constexpr (SPLITK) {  // raw partial sums of this split; the epilogue runs in splitk_epilogue_kernel
          if (!valid) continue;
          float* prow = g.part + ((int64_t)(t % splits) * g.M + (c.m0 + r)) * g.N + nb;
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (nb + j < g.N) prow[j] = __uint_as_float(v[j]) + __uint_as_float(u[j]);
          continue;
        }
        if (!g.store_mode && !valid) continue;
        float o[32];
#pragma unroll
        for (int j = 0; j < 32; j++) {
          float x = __uint_as_float(v[j]) + __uint_as_float(u[j]);
          if ((g.flags & OMT_EPI_BIAS) && nb + j < g.N) x += __ldg(g.bias + nb + j);
          if (g.flags & OMT_EPI_RELU) x = fmaxf(x, 0.f);
          o[j] = x;
        }
        if (g.store_mode) {
          if (dbg & 1) continue;
          if (lane == 0 && !(dbg & 2)) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the previous box has left the buffer
          __syncwarp();
          float4* row = reinterpret_cast<float4*>(buf + lane * 128);
#pragma unroll
          for (int j = 0; j < 8; j++) row[j ^ (lane & 7)] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (g.store_mode == 1) {
              if (g.flags & OMT_EPI_ACCUM) tma_reduce_add_2d(&map_y, smem_u32(buf), nb, c.m0 + q * 32);
              else tma_store_2d(&map_y, smem_u32(buf), nb, c.m0 + q * 32);
            } else {
              const int r0 = q * 32;
              tma_store_4d(&map_y, smem_u32(buf), nb, c.ox0 + r0 % win_w, c.oy0 + r0 / win_w, c.img0);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          if (g.flags & OMT_EPI_BNSTATS) {
            // Batch-norm statistics of what was just stored, from the box in shared memory (the TMA store only reads it):
            // lane l takes channel nb + l, i.e. column l of the 32 rows, whose 16-byte slot in row r is (l / 4) ^ (r & 7), so
            // the 32 lanes of one load hit 32 different banks. One pass, shifted by the group's first valid row (the
            // deviations are then of the order of the spread, whatever the mean).
            const uint32_t vmask = __ballot_sync(0xffffffffu, valid);
            const int cnt = __popc(vmask);
            const int grp = (t / n_tiles) * 4 + q;
            float s1 = 0.f, s2 = 0.f, shift = 0.f;
            if (cnt) {
              const int r0 = __ffs(vmask) - 1;
              shift = *reinterpret_cast<const float*>(buf + r0 * 128 + ((((lane >> 2) ^ (r0 & 7)) << 4) | ((lane & 3) << 2)));
              float p1[4] = {0.f, 0.f, 0.f, 0.f}, p2[4] = {0.f, 0.f, 0.f, 0.f};  // four independent chains (fixed order: deterministic)
#pragma unroll
              for (int r = 0; r < 32; r++) {
                const float v = *reinterpret_cast<const float*>(buf + r * 128 + ((((lane >> 2) ^ (r & 7)) << 4) | ((lane & 3) << 2)));
                const float d = ((vmask >> r) & 1u) ? v - shift : 0.f;
                p1[r & 3] += d; p2[r & 3] = fmaf(d, d, p2[r & 3]);
              }
              s1 = (p1[0] + p1[1]) + (p1[2] + p1[3]); s2 = (p2[0] + p2[1]) + (p2[2] + p2[3]);
            }
            if (nb + lane < g.N) {
              const float fc = (float)cnt;
              g.stats[((int64_t)2 * grp) * g.N + nb + lane] = fmaf(fc, shift, s1);                          // sum of the group
              g.stats[((int64_t)2 * grp + 1) * g.N + nb + lane] = cnt ? fmaxf(s2 - s1 * s1 / fc, 0.f) : 0.f;  // sum (v - group mean)^2
            }
            if (nb == 0 && lane == 0) g.stats[(int64_t)2 * m_tiles * 4 * g.N + grp] = (float)cnt;
            // ticket counters of the kernel that merges the partials (one per 32 channels), behind the counts
            if (grp == 0 && lane == 0) g.stats[(int64_t)m_tiles * 4 * (2 * g.N + 1) + (nb >> 5)] = 0.f;
          }
        } else if (g.flags & OMT_EPI_ACCUM) {  // every output element belongs to exactly one tile row: a plain read-add-write
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (nb + j < g.N) yrow[(int64_t)(nb + j) * g.y.sc] += o[j];
        } else if (vec && nb + 32 <= g.N) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(yrow + nb + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (nb + j < g.N) yrow[(int64_t)(nb + j) * g.y.sc] = o[j];
        }
      }
      // hand the accumulator pair back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(LEADER(ACC_EMPTY + b));
        else mbar_arrive(BAR(ACC_EMPTY + b));
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every box this warp stored has been written
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // neither CTA leaves (or frees TMEM) while the other may still signal it or read its tiles
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// weight re-layout: w[co][ci][ks][ks] -> out[2][rows][kh*kw][cpad], hi and lo planes, zero padded
//   forward:  rows = co, channel = ci, tap (ty, tx) reads w[.., ty, tx]                       (kh = kw = ks)
//   dgrad:    rows = ci, channel = co, tap (ty, tx) reads w[.., ky0 + step*(kh-1-ty), kx0 + step*(kw-1-tx)]
//             (transposed and flipped; for a strided convolution one call per stride phase with that phase's taps)
// ---------------------------------------------------------------------------------------------------------------------
struct SplitArgs {
  int co, ci, ks, kh, kw, cpad, dgrad, ky0, kx0, step;
  int window;  // forward, window mode: tap = filter row ky, column k' = kx*4 + c
};
__global__ void __launch_bounds__(256) weight_split_kernel(const float* __restrict__ w, float* __restrict__ out, SplitArgs a) {
  const int rows = a.dgrad ? a.ci : a.co, chans = a.window ? a.cpad : (a.dgrad ? a.co : a.ci), kk = a.kh * a.kw;
  const int64_t total = (int64_t)rows * kk * a.cpad;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = (int)(i % a.cpad);
  const int tap = (int)((i / a.cpad) % kk);
  const int row = (int)(i / ((int64_t)a.cpad * kk));
  float v = 0.f;
  if (c < chans) {
    int ty = tap / a.kw, tx = tap - ty * a.kw;
    if (a.window) {
      int kx = c >> 2, cc = c & 3;
      v = (kx < a.ks && cc < a.ci) ? __ldg(w + (((int64_t)row * a.ci + cc) * a.ks + ty) * a.ks + kx) : 0.f;
    } else if (a.dgrad) {
      int ky = a.ky0 + a.step * (a.kh - 1 - ty), kx = a.kx0 + a.step * (a.kw - 1 - tx);
      v = __ldg(w + (((int64_t)c * a.ci + row) * a.ks + ky) * a.ks + kx);
    } else {
      v = __ldg(w + (((int64_t)row * a.ci + c) * a.ks + ty) * a.ks + tx);
    }
  }
  const float hi = tf32_rna(v);
  out[i] = hi;
  out[total + i] = tf32_rna(v - hi);
}

// ---------------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;
EncodeIm2colFn g_encode_im2col = nullptr;
std::once_flag g_driver_once;

bool load_driver_entry_points() {
  std::call_once(g_driver_once, [] {
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      g_encode_tiled = (EncodeTiledFn)fn;
    fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      g_encode_im2col = (EncodeIm2colFn)fn;
    (void)cudaGetLastError();
  });
  return g_encode_tiled && g_encode_im2col;
}

struct TcProblem {  // a convolution of a channels-last activation `a` [n, ih, iw, c] producing a [n, oh, ow, rows] pixel grid
  const float* a;
  int n, c, ih, iw, oh, ow, rows;
  int kh, kw, stride;
  int low_h, low_w;              // input coordinate of tap (0,0) at output pixel (0,0)
  int out_step, out_y0, out_x0;  // where GEMM row (oy, ox) lands in the output tensor
};

int pick_bn(const TcProblem& p) {
  if (tl_plan.bn == 64 || tl_plan.bn == 128 || tl_plan.bn == 256) return tl_plan.bn;  // tuned or loaded for this geometry
  if (p.rows <= 64) return 64;
  if (p.rows <= 128) return 128;
  // (128 x 256 tiles with a short reduction use one accumulator per tile and two TMEM buffers, so their epilogue overlaps the
  // next tile like that of the 128 x 128 tiles, and A is read half as often: measured 0.344 -> 0.295 ms on 64 -> 256 1x1 at 56^2)
  int64_t mt = cdiv((int64_t)p.n * p.oh * p.ow, BM);
  if (mt * cdiv(p.rows, 256) < sm_count()) return 128;
  // tile quantisation: rounds of the persistent loop with either width; a 128 x 256 tile costs about 1.8 tiles of 128 x 128
  // (e.g. 196 tiles of 256 columns on 148 SMs pay 2 rounds for 1.3; 392 of 128 columns pay 3 for 2.6)
  const int64_t r256 = cdiv(mt * cdiv(p.rows, 256), sm_count()), r128 = cdiv(mt * cdiv(p.rows, 128), sm_count());
  return 10 * r128 < 18 * r256 ? 128 : 256;
}

// split-K plan: only when the output tiles leave most SMs idle and the reduction is long enough to share
int plan_splits(int64_t M, int64_t N, int kblocks, int bn) {
  const int64_t tiles = cdiv(M, BM) * cdiv(N, bn);
  if (tiles * 2 > sm_count() || kblocks < 8) return 1;
  return (int)std::max<int64_t>(1, std::min<int64_t>(kblocks / 4, sm_count() / tiles));
}

// y(m, n) = epilogue(sum over splits of part[s][m][n]) for the GEMM row m = (img, oy, ox) of the (sub-)convolution
__global__ void __launch_bounds__(256) splitk_epilogue_kernel(TcArgs g) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)g.M * g.N) return;
  const int n = (int)(i % g.N);
  const int m = (int)(i / g.N);
  float v = 0.f;
  for (int s = 0; s < g.splits; s++) v += __ldg(g.part + ((int64_t)s * g.M + m) * g.N + n);
  if (g.flags & OMT_EPI_BIAS) v += __ldg(g.bias + n);
  if (g.flags & OMT_EPI_RELU) v = fmaxf(v, 0.f);
  const int ohw = g.oh * g.ow, img = m / ohw, rr = m - img * ohw, oy = rr / g.ow, ox = rr - oy * g.ow;
  float* dst = g.y.p + g.y.off(img, n, oy * g.out_step + g.out_y0, ox * g.out_step + g.out_x0);
  if (g.flags & OMT_EPI_ACCUM) *dst += v;
  else *dst = v;
}

// dense channels-last output written pixel for pixel (no phase stride), 16-byte aligned rows
bool dense_out(const TcArgs& a) {
  const ActView& y = a.y;
  return a.out_step == 1 && a.out_y0 == 0 && a.out_x0 == 0 && y.sc == 1 && (a.ow == 1 || y.sw == a.N) && (a.oh == 1 || y.sh == (int64_t)a.ow * a.N) &&
         y.sn == (int64_t)a.oh * a.ow * a.N && a.N % 4 == 0 && (reinterpret_cast<uintptr_t>(y.p) & 15) == 0;
}

// OMARCHY_MAC_TORCH_CTA_PAIRS (read once): 0 = no CTA pairs, 1 (default) = in the weight gradient, 2 = also in forward / input
// gradient. Measured on the ResNet-50 step: with the a_hi products issued ahead of the split, single-CTA forward / input
// gradient tiles take 25.3 ms per step against 26.0 ms for pairs (which cannot issue ahead: rank 0 learns that the other
// CTA's A tile has landed only through its split warps); the weight gradient takes 15.0 ms with pairs against 15.5.
static int cta_pairs_mode() {
  static const int mode = [] {
    const char* e = getenv("OMARCHY_MAC_TORCH_CTA_PAIRS");
    return e && e[0] >= '0' && e[0] <= '2' ? e[0] - '0' : 1;
  }();
  return mode;
}
static bool cta_pairs_enabled() { return cta_pairs_mode() >= 1; }
static_assert(Smem<64, false, false, true>::TOTAL == Smem<64>::TOTAL, "both 64-column kernels are launched with the same shared-memory size");
// the weight gradient of 3x3 layers with at most 64 output channels pairs taps unless OMARCHY_MAC_TORCH_TAP_PAIRS=0 (read once)
static bool tap_pairs_enabled() {
  static const bool on = [] {
    const char* e = getenv("OMARCHY_MAC_TORCH_TAP_PAIRS");
    return !(e && e[0] == '0');
  }();
  return on;
}
// 64-column tiles take their A_lo operand from tensor memory unless OMARCHY_MAC_TORCH_A_TMEM=0 (read once)
static bool a_tmem_enabled() {
  static const bool on = [] {
    const char* e = getenv("OMARCHY_MAC_TORCH_A_TMEM");
    return !(e && e[0] == '0');
  }();
  return on;
}
// clusters of two CTAs of the pair kernel that can be resident at once (0: the launch form is not available), once per instantiation
template <int BN, bool ACC1>
static int pair_clusters() {
  using SP = Smem<BN, ACC1, true>;
  static std::once_flag once;
  static int clusters = 0;
  std::call_once(once, [] {
    auto kernel = conv_tc_kernel<BN, false, ACC1, true>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SP::TOTAL) != cudaSuccess) { cudaGetLastError(); return; }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(sm_count() & ~1)); cfg.blockDim = dim3(TC_THREADS); cfg.dynamicSmemBytes = SP::TOTAL;
    cudaLaunchAttribute at{};
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); return; }
    clusters = std::min(n, sm_count() / 2);
  });
  return clusters;
}
template <int BN, bool ACC1>
static int launch_pair(const CUtensorMap& map_a, const CUtensorMap& map_w, const CUtensorMap& map_y, const TcArgs& a, int clusters, cudaStream_t s) {
  using SP = Smem<BN, ACC1, true>;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2u * (unsigned)clusters); cfg.blockDim = dim3(TC_THREADS); cfg.dynamicSmemBytes = SP::TOTAL; cfg.stream = s;
  cudaLaunchAttribute at{};
  at.id = cudaLaunchAttributeClusterDimension;
  at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
  cfg.attrs = &at; cfg.numAttrs = 1;
  OMT_CUDA(cudaLaunchKernelEx(&cfg, conv_tc_kernel<BN, false, ACC1, true>, map_a, map_w, map_y, a));
  return check_launch(BN == 64 ? "conv_tc_256x64_pair" : (BN == 128 ? "conv_tc_256x128_pair" : (ACC1 ? "conv_tc_256x256_pair_acc1" : "conv_tc_256x256_pair")));
}

template <int BN>
int launch_tc(const TcProblem& p, const float* wsplit, const TcArgs& args, int splits, float* part, cudaStream_t s) {
  using S = Smem<BN>;
  alignas(64) CUtensorMap map_a, map_w;
  // 128 x 256 tiles with a short reduction: one accumulator per tile, so that two tiles fit TMEM and the epilogue overlaps
  const bool acc1 = BN == 256 && splits == 1 && p.kh * p.kw * args.cblocks <= ACC1_MAX_KBLOCKS && !(args.flags & OMT_PRECISE_ACCUM);
  // two CTAs per 256 x 256 tile pair when the row tiles pair up (each CTA then stages half of the weight tile)
  int clusters = 0;
  // (only the 256-column tiles: measured on 64- and 128-column tiles, pairs lose 30-40 % -- they give up the double-width MMA
  // over [B_hi; B_lo] and pay the cross-SM barrier round trip on stages that are short already)
  if (BN == 256 && splits == 1 && cdiv(args.M, BM) % 2 == 0 && p.kh * p.kw * args.cblocks >= PAIR_MIN_KBLOCKS && cta_pairs_mode() >= 2)
    clusters = acc1 ? pair_clusters<256, true>() : pair_clusters<256, false>();
  const bool pair = clusters > 0;
  {
    cuuint64_t dims[4] = {(cuuint64_t)p.c, (cuuint64_t)p.iw, (cuuint64_t)p.ih, (cuuint64_t)p.n};
    cuuint64_t strides[3] = {(cuuint64_t)p.c * 4, (cuuint64_t)p.iw * p.c * 4, (cuuint64_t)p.ih * p.iw * p.c * 4};
    // base pixels run over [low, dim - 1 + upper] in steps of `stride`; their count must equal the output extent
    int lower[2] = {p.low_w, p.low_h};
    int upper[2] = {(p.ow - 1) * p.stride + p.low_w - (p.iw - 1), (p.oh - 1) * p.stride + p.low_h - (p.ih - 1)};
    cuuint32_t estr[4] = {1, (cuuint32_t)p.stride, (cuuint32_t)p.stride, 1};
    CUresult r = g_encode_im2col(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)p.a, dims, strides, lower, upper, BKF, BM, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("cuTensorMapEncodeIm2col failed (%d) for corners (%d,%d)/(%d,%d)", (int)r, lower[0], lower[1], upper[0], upper[1]);
      return OMT_ECUDA;
    }
  }
  {
    const int kp = p.kh * p.kw * args.cblocks * BKF;
    cuuint64_t dims[3] = {(cuuint64_t)kp, (cuuint64_t)p.rows, 2};
    cuuint64_t strides[2] = {(cuuint64_t)kp * 4, (cuuint64_t)kp * 4 * p.rows};
    cuuint32_t box[3] = {BKF, (cuuint32_t)(pair ? BN / 2 : BN), 1}, estr[3] = {1, 1, 1};
    CUresult r = g_encode_tiled(&map_w, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)wsplit, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("cuTensorMapEncodeTiled failed (%d)", (int)r);
      return OMT_ECUDA;
    }
  }
  // once per instantiation, from whichever thread gets here first (autograd's worker threads call these too)
  static std::once_flag attr_once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once, [] {
    attr_err = cudaFuncSetAttribute((conv_tc_kernel<BN, false>), cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute((conv_tc_kernel<BN, true>), cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (attr_err == cudaSuccess && BN == 256)
      attr_err = cudaFuncSetAttribute((conv_tc_kernel<BN, false, BN == 256>), cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (attr_err == cudaSuccess && BN == 64)
      attr_err = cudaFuncSetAttribute((conv_tc_kernel<BN, false, false, false, BN == 64>), cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
  });
  OMT_CUDA(attr_err);
  TcArgs a = args;
#ifdef OMT_TC_EXPERIMENTS
  if (const char* e = getenv("OMT_TC_DBG")) a.reserved_[0] = atoi(e);
#endif
  alignas(64) CUtensorMap map_y = map_w;  // placeholder when the epilogue stores directly
  if (splits > 1) {  // partial tiles go to the workspace with plain stores (these fields alias the window fields, unused here)
    a.splits = splits; a.unused_ = 0; a.part = part;
  } else if (dense_out(a)) {  // the output is the row-major [M, N] matrix: 32 x 32 boxes leave through TMA
    cuuint64_t dims[2] = {(cuuint64_t)a.N, (cuuint64_t)a.M};
    cuuint64_t strides[1] = {(cuuint64_t)a.N * 4};
    cuuint32_t box[2] = {32, 32}, estr[2] = {1, 1};
    if (g_encode_tiled(&map_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)a.y.p, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
      a.store_mode = 1;
  }
  // the statistics are taken from the 32 x 32 boxes staged for the TMA stores, by the kernel that owns the whole reduction
  OMT_REQUIRE(!(a.flags & OMT_EPI_BNSTATS) || a.store_mode == 1, "OMT_EPI_BNSTATS needs a dense channels-last output and an unsplit reduction");
  const int m_tiles = (int)cdiv(a.M, BM), n_tiles = (int)cdiv(a.N, BN);
  const unsigned grid = (unsigned)std::min<int64_t>((int64_t)m_tiles * n_tiles * splits, sm_count());
  if (pair) {
    const int work = (m_tiles / 2) * n_tiles;
    return acc1 ? launch_pair<256, true>(map_a, map_w, map_y, a, std::min(work, clusters), s)
                : launch_pair<256, false>(map_a, map_w, map_y, a, std::min(work, clusters), s);
  }
  if (splits > 1) conv_tc_kernel<BN, true><<<grid, TC_THREADS, S::TOTAL, s>>>(map_a, map_w, map_y, a);
  else if (acc1) conv_tc_kernel<BN, false, BN == 256><<<grid, TC_THREADS, S::TOTAL, s>>>(map_a, map_w, map_y, a);
  else if (BN == 64 && a_tmem_enabled()) conv_tc_kernel<BN, false, false, false, BN == 64><<<grid, TC_THREADS, S::TOTAL, s>>>(map_a, map_w, map_y, a);
  else conv_tc_kernel<BN, false><<<grid, TC_THREADS, S::TOTAL, s>>>(map_a, map_w, map_y, a);
  int r = check_launch(BN == 64 ? (splits == 1 && a_tmem_enabled() ? "conv_tc_128x64_atmem" : "conv_tc_128x64") : (BN == 128 ? "conv_tc_128x128" : (acc1 ? "conv_tc_128x256_acc1" : "conv_tc_128x256")));
  if (r || splits == 1) return r;
  splitk_epilogue_kernel<<<(unsigned)cdiv((int64_t)a.M * a.N, 256), 256, 0, s>>>(a);
  return check_launch("conv_tc_splitk_epilogue");
}

size_t split_floats(int rows, int ks, int chans) { return (size_t)2 * rows * ks * ks * (cdiv(chans, BKF) * BKF); }

// one (sub-)convolution: re-lay the weights it needs into `wsplit`, then run the GEMM
int run_tc(const TcProblem& p, const float* w, SplitArgs sp, float* wsplit, float* part, const OmtAct* y, const float* bias, float* stats,
           uint32_t flags, cudaStream_t s) {
  TcArgs a{};
  a.y = view(y); a.bias = bias;
  a.M = p.n * p.oh * p.ow; a.N = p.rows; a.oh = p.oh; a.ow = p.ow;
  a.kh = (int16_t)p.kh; a.kw = (int16_t)p.kw; a.stride = (int8_t)p.stride; a.low_h = p.low_h; a.low_w = p.low_w;
  a.out_step = (int8_t)p.out_step; a.out_y0 = (int8_t)p.out_y0; a.out_x0 = (int8_t)p.out_x0;
  a.cblocks = (int)cdiv(p.c, BKF);
  a.flags = flags; a.stats = stats;
  const int cpad = a.cblocks * BKF;
  sp.kh = p.kh; sp.kw = p.kw; sp.cpad = cpad;
  const int64_t total = (int64_t)p.rows * p.kh * p.kw * cpad;
  weight_split_kernel<<<(unsigned)cdiv(total, 256), 256, 0, s>>>(w, wsplit, sp);
  int r = check_launch("conv_tc_weight_split");
  if (r) return r;
  const int bn = pick_bn(p);
  const int splits = plan_splits(a.M, a.N, p.kh * p.kw * a.cblocks, bn);
  switch (bn) {
    case 64: return launch_tc<64>(p, wsplit, a, splits, part, s);
    case 128: return launch_tc<128>(p, wsplit, a, splits, part, s);
    default: return launch_tc<256>(p, wsplit, a, splits, part, s);
  }
}
// floats of split-K partial tiles this (sub-)convolution needs (0 when it does not split)
size_t part_floats(const TcProblem& p) {
  const int64_t M = (int64_t)p.n * p.oh * p.ow;
  const int splits = plan_splits(M, p.rows, p.kh * p.kw * (int)cdiv(p.c, BKF), pick_bn(p));
  return splits > 1 ? (size_t)splits * M * p.rows : 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// weight gradient kernel
// ---------------------------------------------------------------------------------------------------------------------
// PB = pixels (reduction depth) per stage, a template parameter: 16 with twice the stages when a stage is one or two TMA boxes
// per operand (covers the load latency better), 32 when a stage needs many boxes (their per-instruction cost dominates)
constexpr int WG_THREADS = 320;   // producer warp, MMA warp, 8 split/epilogue warps

struct WgArgs {
  // bit 0: gy tile by one 3-D TMA box; bit 1: x is the plain [pixels, ci] matrix (1x1, stride 1), one 3-D box.
  // bit 2: "rectangle" pixel blocks: a stage holds bw x bh pixels of bn images (bw*bh*bn = 32) so that both operands come
  //        through tiled tensor maps, gy as one 5-D box and x as one 5-D box per filter tap (`cpi` 32-channel blocks each),
  //        shifted by the tap and zero-filled outside the image.
  // bit 3: with bit 2, "window" x operand for <= 4 input channels: the 32-float run (8 pixels x 4 channels) of a filter
  //        row out of the padded 4-channel staging copy, one box per (filter row, 32-float block) chunk; bw = 32.
  // bit 4: with bit 2, "paired taps" for co <= 64: the lower half of the 128-row gy tile would be empty, so it holds gy
  //        shifted by one pixel (shift_x) or one row (shift_y), zero outside the image, and every x column gives two taps:
  //        sum_p gy[p + 1] x[p * stride + k] = sum_q gy[q] x[q * stride + (k - stride)]. The tile's columns run over the
  //        taps `top[v]` only ("virtual" chunks, `chunks`); the epilogue writes rows 0-63 to the columns of top[v] and rows
  //        64-127 to those of bot[v] (< 0: none). The q = 0 term of the second sum has no p: it must multiply padding
  //        (3x3, stride 1, pad 1 pairing (ky, 1) with (ky, 0)), or the pixel blocks start one row above the image
  //        (shift_y; window mode, where top/bot are filter rows).
  int mode;
  int total_blocks;  // pixel blocks in all
  int bw, bh, bn, tiles_x, tiles_y, cpi;
  float* part;       // [slices][co][kcols] partial tiles
  int P;             // pixels = n * oh * ow
  int co;
  int oh, ow, ks, stride, pad;
  int cblocks, cpad; // 32-channel blocks per tap
  int chunks;        // ks * ks * cblocks: 32-wide column chunks of the output (paired taps: 6 * cblocks, the columns computed)
  int out_chunks;    // 32-wide column chunks of a row of `part`
  int8_t top[16], bot[16];
  int8_t shift_x, shift_y;
  int blocks_per_slice;  // 32-pixel blocks per blockIdx.z
};

// PAIR: the CTA is one of a cta_group::2 pair (two 128-row co tiles, one stream of 256-row MMAs) and stages only its half of
// the x columns; the smaller stages leave room for a deeper ring.
template <int BN, int PB, bool PAIR = false>
struct WgSmem {
  static constexpr int TMEM_COLS = 2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512);  // main + cross-term accumulators, a power of two
  static constexpr int CH = PB * 128;                 // one 32-pixel x 32-float box
  static constexpr int B_CHUNKS = BN / 32 / (PAIR ? 2 : 1);  // 32-column chunks of x this CTA stages
  static constexpr int A_BYTES = 4 * CH, B_BYTES = B_CHUNKS * CH;
  static constexpr int HALF = A_BYTES + B_BYTES;      // hi region; the lo region follows at +HALF
  static constexpr int STAGE_BYTES = 2 * HALF;
  static constexpr int STAGES = PAIR ? (200 * 1024 / STAGE_BYTES < 8 ? 200 * 1024 / STAGE_BYTES : 8) : (BN >= 192 ? 2 : (BN == 128 ? 3 : 4)) * (32 / PB);
  static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// PAIR (clusters of two CTAs along blockIdx.x, i.e. two neighbouring co tiles of the same columns and slice): each CTA loads
// and splits its own gy rows and HALF of the x chunks; the split warps of both arrive on CTA rank 0's "split" barrier, whose
// MMA thread issues tcgen05.mma.cta_group::2 (M = 256) for both and signals "free" / "accumulator ready" in both CTAs with
// multicast commits. Both operands are split on the fly here, so halving the x side removes a third of a stage's
// shared-memory traffic (the single-CTA kernel is bound by it).
template <int BN, int PB, bool PAIR = false>
__global__ void __launch_bounds__(WG_THREADS, 1)
wgrad_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_g, const WgArgs g) {
  using S = WgSmem<BN, PB, PAIR>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::BAR_OFF);
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * i; };  // [0,S) loaded, [S,2S) split, [2S,3S) free, 3S accumulator ready
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 3 * S::STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 3 * S::STAGES + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int co0 = blockIdx.x * BM;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int nchunks = min(BN / 32, g.chunks - (int)blockIdx.y * (BN / 32));  // columns of the tile (the epilogue's view)
  const int nown = PAIR ? S::B_CHUNKS : nchunks;                               // x chunks this CTA loads (pairs take full tiles only)
  const int chunk0 = blockIdx.y * (BN / 32) + (int)rank * (PAIR ? S::B_CHUNKS : 0);
  auto LEADER = [&](int i) { return PAIR ? mapa_rank(BAR(i), 0u) : BAR(i); };
  const int total_blocks = g.total_blocks;
  const int blk_begin = blockIdx.z * g.blocks_per_slice;
  const int kblocks = max(0, min(g.blocks_per_slice, total_blocks - blk_begin));

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; s++) {
      mbar_init(BAR(s), 1);
      mbar_init(BAR(S::STAGES + s), PAIR ? 16 : 8);  // the split warps (of both CTAs of a pair)
      mbar_init(BAR(2 * S::STAGES + s), 1);
    }
    mbar_init(BAR(3 * S::STAGES), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                   "r"((uint32_t)S::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                   "r"((uint32_t)S::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const int ohw = g.oh * g.ow;
      int issued = 0;
      for (int kb = 0; kb < kblocks; kb++) {
        const int s = kb % S::STAGES, round = kb / S::STAGES;
        if (round > 0 && !mbar_wait(BAR(2 * S::STAGES + s), (round - 1) & 1, abort_flag)) break;
        const uint32_t stage = smem_base + s * S::STAGE_BYTES;
        if (g.mode & 4) {
          const int b = blk_begin + kb;
          const int tx = b % g.tiles_x, r1 = b / g.tiles_x, ty = r1 % g.tiles_y, tn = r1 / g.tiles_y;
          const int ox0 = tx * g.bw, oy0 = ty * g.bh - ((g.mode & 16) ? g.shift_y : 0), n0 = tn * g.bn;
          mbar_expect_tx(BAR(s), S::A_BYTES + nown * S::CH);
          if (g.mode & 16) {  // two boxes of two channel blocks: gy, and gy one pixel to the right / one row down
            tma_tile_5d(stage, &map_g, BAR(s), 0, ox0, oy0, n0, 0);
            tma_tile_5d(stage + 2 * S::CH, &map_g, BAR(s), 0, ox0 + g.shift_x, oy0 + g.shift_y, n0, 0);
          } else {
            tma_tile_5d(stage, &map_g, BAR(s), 0, ox0, oy0, n0, co0 / 32);
          }
          if (g.mode & 8) {
            for (int j = 0; j < nown; j++) {
              const int chunk = chunk0 + j, v = chunk / g.cblocks, blk = chunk - v * g.cblocks;
              const int ky = (g.mode & 16) ? g.top[v] : v;
              tma_tile_4d(stage + S::A_BYTES + j * S::CH, &map_x, BAR(s), blk * BKF, ox0, oy0 * g.stride + ky - g.pad, n0);
            }
          } else {
            for (int j = 0; j < nown; j += g.cpi) {
              const int chunk = chunk0 + j, v = chunk / g.cblocks, cb = chunk - v * g.cblocks;
              const int tap = (g.mode & 16) ? g.top[v] : v, ky = tap / g.ks, kx = tap - ky * g.ks;
              tma_tile_5d(stage + S::A_BYTES + j * S::CH, &map_x, BAR(s), 0, ox0 * g.stride - g.pad + kx, oy0 * g.stride - g.pad + ky, n0, cb);
            }
          }
          issued = kb + 1;
          continue;
        }
        const int p0 = (blk_begin + kb) * PB;
        const int img = p0 / ohw, r = p0 - img * ohw, oy = r / g.ow, ox = r - oy * g.ow;
        const int w0 = ox * g.stride - g.pad, h0 = oy * g.stride - g.pad;
        mbar_expect_tx(BAR(s), S::A_BYTES + ((g.mode & 2) ? S::B_BYTES : nown * S::CH));
        if (g.mode & 1) {
          tma_tile_3d(stage, &map_g, BAR(s), 0, p0, co0 / 32);
        } else {
#pragma unroll
          for (int i = 0; i < 4; i++) tma_tile_2d(stage + i * S::CH, &map_g, BAR(s), co0 + 32 * i, p0);
        }
        if (g.mode & 2) {
          tma_tile_3d(stage + S::A_BYTES, &map_x, BAR(s), 0, p0, chunk0);
        } else {
          for (int j = 0; j < nown; j++) {
            const int chunk = chunk0 + j, tap = chunk / g.cblocks, cb = chunk - tap * g.cblocks;
            const int ky = tap / g.ks, kx = tap - ky * g.ks;
            tma_im2col_4d(stage + S::A_BYTES + j * S::CH, &map_x, BAR(s), cb * BKF, w0, h0, img, (uint16_t)kx, (uint16_t)ky);
          }
        }
        issued = kb + 1;
      }
      if (*abort_flag) {
        for (int kb = max(0, issued - S::STAGES); kb < issued; kb++) {
          const long long t0 = clock64();
          while (!mbar_try(BAR(kb % S::STAGES), (kb / S::STAGES) & 1) && clock64() - t0 < WAIT_BUDGET_CLOCKS) {}
        }
      } else if (PAIR) {  // the last "free" arrivals come from the other SM's commit: let them land before this CTA exits
        for (int kb = max(0, issued - S::STAGES); kb < issued; kb++)
          if (!mbar_wait(BAR(2 * S::STAGES + kb % S::STAGES), (kb / S::STAGES) & 1, abort_flag)) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_tf32(BN, true, PAIR ? 2 * BM : BM);
      auto umma_tf32 = [](uint32_t d, uint64_t da, uint64_t db, uint32_t id, uint32_t accumulate) {
        if constexpr (PAIR) umma_tf32_pair(d, da, db, id, accumulate);
        else omt::umma_tf32(d, da, db, id, accumulate);
      };
      auto umma_commit = [](uint32_t bar) {
        if constexpr (PAIR) umma_commit_pair(bar);
        else omt::umma_commit(bar);
      };
      bool ok = true;
      for (int kb = 0; kb < kblocks && ok; kb++) {
        const int s = kb % S::STAGES, round = kb / S::STAGES;
        // (a pair's "split" barrier counts the split warps of both CTAs, each of which waited for its own loads)
        const uint32_t stage = smem_base + s * S::STAGE_BYTES;
        if constexpr (!PAIR) {
          // one CTA: a_hi x b_hi needs only what TMA loaded and is issued while the split warps still work on the stage
          ok = mbar_wait(BAR(s), round & 1, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int k = 0; k < PB / UMMA_K; k++) {
            const uint32_t koff = k * 1024;
            umma_tf32(tmem_acc, smem_desc_mn_sw128(stage + koff, S::CH), smem_desc_mn_sw128(stage + S::A_BYTES + koff, S::CH), idesc, (kb | k) ? 1u : 0u);
          }
          ok = mbar_wait(BAR(S::STAGES + s), round & 1, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int k = 0; k < PB / UMMA_K; k++) {
            const uint32_t koff = k * 1024;
            const uint64_t a_hi = smem_desc_mn_sw128(stage + koff, S::CH), a_lo = smem_desc_mn_sw128(stage + S::HALF + koff, S::CH);
            const uint64_t b_hi = smem_desc_mn_sw128(stage + S::A_BYTES + koff, S::CH);
            const uint64_t b_lo = smem_desc_mn_sw128(stage + S::HALF + S::A_BYTES + koff, S::CH);
            umma_tf32(tmem_acc + BN, a_lo, b_hi, idesc, (kb | k) ? 1u : 0u);  // cross terms in their own accumulator
            umma_tf32(tmem_acc + BN, a_hi, b_lo, idesc, 1u);
          }
          umma_commit(BAR(2 * S::STAGES + s));
          continue;
        }
        ok = mbar_wait<PAIR>(BAR(S::STAGES + s), round & 1, abort_flag) && (PAIR || mbar_wait(BAR(s), round & 1, abort_flag));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int k = 0; k < PB / UMMA_K; k++) {
          const uint32_t koff = k * 1024;  // next group of 8 pixel rows
          const uint64_t a_hi = smem_desc_mn_sw128(stage + koff, S::CH), a_lo = smem_desc_mn_sw128(stage + S::HALF + koff, S::CH);
          const uint64_t b_hi = smem_desc_mn_sw128(stage + S::A_BYTES + koff, S::CH);
          const uint64_t b_lo = smem_desc_mn_sw128(stage + S::HALF + S::A_BYTES + koff, S::CH);
          umma_tf32(tmem_acc + BN, a_lo, b_hi, idesc, (kb | k) ? 1u : 0u);  // cross terms in their own accumulator
          umma_tf32(tmem_acc + BN, a_hi, b_lo, idesc, 1u);
          umma_tf32(tmem_acc, a_hi, b_hi, idesc, (kb | k) ? 1u : 0u);
        }
        umma_commit(BAR(2 * S::STAGES + s));
      }
      if (ok) umma_commit(BAR(3 * S::STAGES));
    }
  } else {
    const int t = threadIdx.x - 64;  // 0..255
    bool ok = true;
    const int n16 = (S::A_BYTES + nown * S::CH) / 16;  // 16-byte words that were loaded this stage
    for (int kb = 0; kb < kblocks && ok; kb++) {
      const int s = kb % S::STAGES, round = kb / S::STAGES;
      ok = mbar_wait(BAR(s), round & 1, abort_flag);
      if (!ok) break;
      uint4* hi = reinterpret_cast<uint4*>(smem + s * S::STAGE_BYTES);
      uint4* lo = reinterpret_cast<uint4*>(smem + s * S::STAGE_BYTES + S::HALF);
      for (int idx = t; idx < n16; idx += 256) {
        uint4 h;
        const uint4 l = split_lo(hi[idx], h);
#if !OMT_TC_IMPLICIT_HI
        hi[idx] = h;
#endif
        lo[idx] = l;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(LEADER(S::STAGES + s));
        else mbar_arrive(BAR(S::STAGES + s));
      }
    }
    // epilogue: warps 2..9; quarter = warp & 3, column half = (warp - 2) / 4
    if (ok && kblocks > 0) ok = mbar_wait(BAR(3 * S::STAGES), 0, abort_flag);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int q = warp & 3, half = (warp - 2) >> 2;
      const bool paired = g.mode & 16;
      const int row = paired ? ((q & 1) * 32 + lane) : (co0 + q * 32 + lane);  // paired taps: rows 64-127 are the same channels again
      const int kcols = g.out_chunks * 32;
      float* prow = g.part + ((int64_t)blockIdx.z * g.co + row) * kcols;
#pragma unroll 1
      for (int c = half; c < BN / 32; c += 2) {
        uint32_t v[32];
        if (kblocks > 0) {
          uint32_t u[32];
          tmem_ld32x2(tmem_acc + ((uint32_t)(q * 32) << 16) + c * 32, tmem_acc + ((uint32_t)(q * 32) << 16) + BN + c * 32, v, u);
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(u[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = 0u;  // a slice with no pixels contributes zeros
        }
        if (row >= g.co || c >= nchunks) continue;
        int out_chunk = (int)blockIdx.y * (BN / 32) + c;  // (chunk0 is this CTA's first LOADED chunk)
        if (paired) {  // rows 0-63 are the tap (or filter row) that was loaded, rows 64-127 the one a gy shift before it
          const int v = out_chunk / g.cblocks, cb = out_chunk - v * g.cblocks, t = q >= 2 ? g.bot[v] : g.top[v];
          if (t < 0) continue;
          out_chunk = t * g.cblocks + cb;
        }
        float4* dst = reinterpret_cast<float4*>(prow + out_chunk * 32);
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          dst[j / 4] = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)S::TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)S::TMEM_COLS) : "memory");
  }
}

// dw[o][c][ky][kx] = scale * sum_z part[z][o][tap*cpad + c]
// window mode (win_ks > 0): column of (c, ky, kx) is (ky*win_kb + kx/8)*32 + (kx%8)*4 + c, kcols = win_ks*win_kb*32
// SL threads share an output: thread `sl` adds slices sl, sl + SL, ... and the SL sums are added in order through shared
// memory -- the same association on every run and every rank. For many slices and few outputs (a 64 x 64 1x1 layer: 4096
// outputs x 148 slices), where one thread per output leaves most SMs idle.
template <int SL>
__global__ void __launch_bounds__(256) wgrad_tc_reduce_kernel(const float* __restrict__ part, float* __restrict__ dw, int co, int ci, int kk,
                                                              int cpad, int slices, float scale, int win_ks, int win_kb) {
  // threads run over (o, tap, c) with c fastest: the slab reads coalesce; the strided writes are 1/slices of the traffic
  constexpr int OUTS = 256 / SL;
  const int local = threadIdx.x % OUTS, sl = threadIdx.x / OUTS;
  const int64_t i = (int64_t)blockIdx.x * OUTS + local;
  const int64_t total = (int64_t)co * ci * kk;
  __shared__ float sums[SL > 1 ? 256 : 1];
  float s = 0.f;
  int c = 0, tap = 0, o = 0;
  if (i < total) {
    c = (int)(i % ci);
    tap = (int)((i / ci) % kk);
    o = (int)(i / ((int64_t)kk * ci));
    int64_t kcols = (int64_t)kk * cpad, col = (int64_t)tap * cpad + c;
    if (win_ks) {
      const int ky = tap / win_ks, kx = tap - ky * win_ks;
      kcols = (int64_t)win_ks * win_kb * 32;
      col = (int64_t)(ky * win_kb + kx / 8) * 32 + (kx % 8) * 4 + c;
    }
    const int64_t slab = (int64_t)co * kcols;
    const float* p = part + (int64_t)o * kcols + col;
#pragma unroll 4
    for (int z = sl; z < slices; z += SL) s += __ldg(p + z * slab);
  }
  if constexpr (SL > 1) {
    sums[threadIdx.x] = s;
    __syncthreads();
    if (sl != 0) return;
#pragma unroll
    for (int j = 1; j < SL; j++) s += sums[j * OUTS + local];
  }
  if (i < total) dw[((int64_t)o * ci + c) * kk + tap] = s * scale;
}
void launch_wgrad_reduce(const float* part, float* dw, int co, int ci, int kk, int cpad, int slices, float scale, int win_ks, int win_kb,
                         cudaStream_t s) {
  const int64_t total = (int64_t)co * ci * kk;
  // (measured per ResNet-50 layer at batch 256: sharing an output among threads pays only for the one-tile layers with a slice
  // per SM, 64 -> 64 1x1 0.148 -> 0.135 ms; with 2-37 slices the plain kernel is as fast or faster)
  if (slices >= 64) wgrad_tc_reduce_kernel<16><<<(unsigned)cdiv(total, 16), 256, 0, s>>>(part, dw, co, ci, kk, cpad, slices, scale, win_ks, win_kb);
  else wgrad_tc_reduce_kernel<1><<<(unsigned)cdiv(total, 256), 256, 0, s>>>(part, dw, co, ci, kk, cpad, slices, scale, win_ks, win_kb);
}

// ---------------------------------------------------------------------------------------------------------------------
// window mode (ci <= 4): staging copy and host side
// ---------------------------------------------------------------------------------------------------------------------
// xs[n][ih][ws][4] = x[n][c][h][w - pad] (zero outside, zero for c >= ci): a channels-last copy padded to 4 channels and
// by `pad` zero pixels on the left (and enough on the right), so that the window rows need no horizontal bounds handling.
__global__ void __launch_bounds__(256) stage_window_kernel(ActView x, float* __restrict__ xs, int n, int ci, int ih, int iw, int ws, int pad) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)n * ih * ws;
  if (i >= total) return;
  const int wp = (int)(i % ws);
  const int h = (int)((i / ws) % ih);
  const int img = (int)(i / ((int64_t)ws * ih));
  const int w = wp - pad;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (w >= 0 && w < iw) {
    const float* p = x.p + x.off(img, 0, h, w);
#pragma unroll
    for (int c = 0; c < 4; c++)
      if (c < ci) v[c] = __ldg(p + c * x.sc);
  }
  reinterpret_cast<float4*>(xs)[i] = make_float4(v[0], v[1], v[2], v[3]);
}

struct WinPlan {
  int kb;       // 32-float blocks per filter row: ceil(ks * 4 / 32)
  int ws;       // padded width of the staging copy
  int win_w, win_h, tiles_x, tiles_y;
  size_t stage_floats, split_floats_;
};
WinPlan plan_window(const OmtConvGeo* g) {
  WinPlan w{};
  w.kb = (int)cdiv(g->ks * 4, BKF);
  w.ws = std::max(g->iw + 2 * g->pad, (g->ow - 1) * g->stride + 8 * w.kb) + 8;
  // widest power-of-two tile row that wastes the fewest pixels
  int best = 8;
  double best_eff = 0;
  for (int tw = 8; tw <= 128; tw *= 2) {
    int th = BM / tw;
    double eff = ((double)g->ow * g->oh) / ((double)cdiv(g->ow, tw) * tw * cdiv(g->oh, th) * th);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = tw; }
  }
  w.win_w = best; w.win_h = BM / best;
  w.tiles_x = (int)cdiv(g->ow, w.win_w); w.tiles_y = (int)cdiv(g->oh, w.win_h);
  w.stage_floats = (size_t)g->n * g->ih * w.ws * 4;
  w.split_floats_ = (size_t)2 * g->co * g->ks * w.kb * BKF;
  return w;
}
bool window_ok(const OmtConvGeo* g) {
  if (g->ci > 4 || g->co < 8 || g->pad >= g->ks) return false;
  // box height (win_h rows at the conv stride) must fit a TMA box
  return 128 * g->stride <= 256 * 8;
}

template <int BN>
int launch_window(const OmtConvGeo* g, const WinPlan& w, const float* xs, const float* wsplit, const TcArgs& args, cudaStream_t s) {
  using S = Smem<BN>;
  alignas(64) CUtensorMap map_a, map_w;
  {
    // dims: k' (floats of a window row), ox (overlapping, one conv stride apart), input row, image
    cuuint64_t dims[4] = {(cuuint64_t)w.kb * BKF, (cuuint64_t)g->ow, (cuuint64_t)g->ih, (cuuint64_t)g->n};
    cuuint64_t strides[3] = {(cuuint64_t)g->stride * 16, (cuuint64_t)w.ws * 16, (cuuint64_t)g->ih * w.ws * 16};
    cuuint32_t box[4] = {BKF, (cuuint32_t)w.win_w, (cuuint32_t)(w.win_h * g->stride), 1};
    cuuint32_t estr[4] = {1, 1, (cuuint32_t)g->stride, 1};
    CUresult r = g_encode_tiled(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)xs, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("cuTensorMapEncodeTiled (window operand) failed (%d)", (int)r);
      return OMT_ECUDA;
    }
  }
  {
    const int kp = g->ks * args.cblocks * BKF;
    cuuint64_t dims[3] = {(cuuint64_t)kp, (cuuint64_t)g->co, 2};
    cuuint64_t strides[2] = {(cuuint64_t)kp * 4, (cuuint64_t)kp * 4 * g->co};
    cuuint32_t box[3] = {BKF, (cuuint32_t)BN, 1}, estr[3] = {1, 1, 1};
    CUresult r = g_encode_tiled(&map_w, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)wsplit, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("cuTensorMapEncodeTiled failed (%d)", (int)r);
      return OMT_ECUDA;
    }
  }
  static std::once_flag attr_once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once, [] {
    attr_err = cudaFuncSetAttribute((conv_tc_kernel<BN, false>), cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (attr_err == cudaSuccess && BN == 64)
      attr_err = cudaFuncSetAttribute((conv_tc_kernel<BN, false, false, false, BN == 64>), cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
  });
  OMT_CUDA(attr_err);
  TcArgs a = args;
  alignas(64) CUtensorMap map_y = map_w;
  if (dense_out(a)) {  // 32-pixel pieces of the tile's rectangle: a row segment, or several short rows
    const int bw = std::min(w.win_w, 32), bh = 32 / bw;
    cuuint64_t dims[4] = {(cuuint64_t)a.N, (cuuint64_t)g->ow, (cuuint64_t)g->oh, (cuuint64_t)g->n};
    cuuint64_t strides[3] = {(cuuint64_t)a.N * 4, (cuuint64_t)g->ow * a.N * 4, (cuuint64_t)g->oh * g->ow * a.N * 4};
    cuuint32_t box[4] = {32, (cuuint32_t)bw, (cuuint32_t)bh, 1}, estr[4] = {1, 1, 1, 1};
    if (g_encode_tiled(&map_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)a.y.p, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
      a.store_mode = 2;
  }
  OMT_REQUIRE(!(a.flags & OMT_EPI_BNSTATS) || a.store_mode == 2, "OMT_EPI_BNSTATS needs a dense channels-last output");
  const int m_tiles = g->n * w.tiles_x * w.tiles_y, n_tiles = (int)cdiv(a.N, BN);
  const unsigned grid = (unsigned)std::min<int64_t>((int64_t)m_tiles * n_tiles, sm_count());
  if (BN == 64 && a_tmem_enabled()) conv_tc_kernel<BN, false, false, false, BN == 64><<<grid, TC_THREADS, S::TOTAL, s>>>(map_a, map_w, map_y, a);
  else conv_tc_kernel<BN, false><<<grid, TC_THREADS, S::TOTAL, s>>>(map_a, map_w, map_y, a);
  return check_launch(BN == 64 ? "conv_tc_window_128x64" : (BN == 128 ? "conv_tc_window_128x128" : "conv_tc_window_128x256"));
}

int run_window_fwd(const OmtConvGeo* g, const OmtAct* x, const float* w, const float* bias, const OmtAct* y, float* stats, uint32_t flags, void* ws,
                   cudaStream_t s) {
  const WinPlan wp = plan_window(g);
  float* xs = (float*)ws;
  float* wsplit = xs + ((wp.stage_floats + 63) / 64) * 64;
  const int64_t total = (int64_t)g->n * g->ih * wp.ws;
  stage_window_kernel<<<(unsigned)cdiv(total, 256), 256, 0, s>>>(view(x), xs, g->n, g->ci, g->ih, g->iw, wp.ws, g->pad);
  int r = check_launch("conv_tc_stage_window");
  if (r) return r;
  TcArgs a{};
  a.y = view(y); a.bias = bias;
  a.M = g->n * g->oh * g->ow; a.N = g->co; a.oh = g->oh; a.ow = g->ow;
  a.kh = (int16_t)g->ks; a.kw = 1; a.stride = (int8_t)g->stride; a.low_h = -g->pad; a.low_w = 0;
  a.out_step = 1; a.out_y0 = 0; a.out_x0 = 0;
  a.cblocks = wp.kb; a.flags = flags; a.stats = stats;
  a.win_w = wp.win_w; a.win_h = wp.win_h; a.tiles_x = wp.tiles_x; a.tiles_y = wp.tiles_y;
  SplitArgs sp{g->co, g->ci, g->ks, g->ks, 1, wp.kb * BKF, 0, 0, 0, 1, 1};
  const int64_t wtotal = (int64_t)g->co * g->ks * wp.kb * BKF;
  weight_split_kernel<<<(unsigned)cdiv(wtotal, 256), 256, 0, s>>>(w, wsplit, sp);
  r = check_launch("conv_tc_weight_split");
  if (r) return r;
  const int bn = g->co <= 64 ? 64 : (g->co <= 128 ? 128 : 256);
  switch (bn) {
    case 64: return launch_window<64>(g, wp, xs, wsplit, a, s);
    case 128: return launch_window<128>(g, wp, xs, wsplit, a, s);
    default: return launch_window<256>(g, wp, xs, wsplit, a, s);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// weight gradient: host side
// ---------------------------------------------------------------------------------------------------------------------
struct WgPlan {
  int bn, slices, blocks_per_slice, cblocks, cpad, chunks;
  int mode, total_blocks, bw, bh, bn_img, tiles_x, tiles_y, cpi;
  int vchunks;          // column chunks the tiles run over: `chunks`, or with paired taps (mode bit 4) those of the taps loaded
  int8_t top[16], bot[16], shift_x, shift_y;  // paired taps: per loaded tap (window mode: filter row) the outputs of the two tile halves
  int pb;               // pixels per stage (16 or 32)
  bool pair;            // clusters of two CTAs (cta_group::2)
  int win_kb;           // window mode: 32-float blocks per filter row
  size_t stage_floats;  // window mode: the padded 4-channel copy of x in front of the partial tiles
  size_t part_floats;
};
WgPlan plan_wgrad(const OmtConvGeo* g) {
  WgPlan w{};
  const bool window = g->ci <= 4;
  if (window) {
    const WinPlan wp = plan_window(g);
    w.win_kb = wp.kb; w.stage_floats = ((wp.stage_floats + 63) / 64) * 64;
    w.cblocks = wp.kb; w.cpad = wp.kb * BKF; w.chunks = g->ks * wp.kb;
  } else {
    w.cblocks = (int)cdiv(g->ci, BKF); w.cpad = w.cblocks * BKF; w.chunks = g->ks * g->ks * w.cblocks;
  }
  // at most 64 output channels leave half of the 128-row tile empty. A 3x3 stride-1 layer fills it with gy shifted by one pixel
  // and computes six taps' columns instead of nine (64 -> 64 3x3 at 56^2, batch 256: 0.74 -> 0.51 ms); the window mode with gy
  // shifted by one row, which pairs filter row ky with ky - stride (7x7 stride 2: rows 6, 5, 2, 1 instead of seven).
  const bool narrow = g->co <= 64 && g->co % 32 == 0 && tap_pairs_enabled();
  const bool paired_taps = narrow && !window && g->ks == 3 && g->stride == 1 && g->pad == 1 && g->ci % 32 == 0;
  const bool paired_rows = narrow && window && g->ks <= 16 && g->stride < g->ks;
  w.vchunks = w.chunks;
  if (paired_taps) {
    for (int ky = 0, v = 0; ky < 3; ky++) {
      w.top[v] = (int8_t)(ky * 3 + 1); w.bot[v++] = (int8_t)(ky * 3);
      w.top[v] = (int8_t)(ky * 3 + 2); w.bot[v++] = -1;
    }
    w.shift_x = 1;
    w.vchunks = 6 * w.cblocks;
  } else if (paired_rows) {  // from the last filter row up: a row nobody yields yet is loaded and yields the row `stride` above it
    bool have[16] = {};
    int v = 0;
    for (int ky = g->ks - 1; ky >= 0; ky--) {
      if (have[ky]) continue;
      w.top[v] = (int8_t)ky; w.bot[v] = (int8_t)(ky - g->stride >= 0 ? ky - g->stride : -1);
      if (ky - g->stride >= 0) have[ky - g->stride] = true;
      v++;
    }
    w.shift_y = 1;
    w.vchunks = v * w.cblocks;
  }
  // tile width: the widest that pads the 32-column chunks (nearly) least (18 chunks of a 64-channel 3x3 layer: 3 x 192 columns,
  // not 3 x 256 with the last tile a quarter full; measured 0.83 -> 0.76 ms there)
  int64_t least = INT64_MAX;
  for (int bn : {64, 128, 192, 256}) least = std::min<int64_t>(least, cdiv(w.vchunks, bn / 32) * bn);
  w.bn = 64;
  for (int bn : {128, 192, 256})  // (a wider tile may pad up to 15 % more: AlexNet conv1's 22 chunks run faster as 3 x 256 than as 11 x 64)
    if (cdiv(w.vchunks, bn / 32) * bn * 100 <= least * 115) w.bn = bn;
  if (tl_plan.bn == 64 || tl_plan.bn == 128 || tl_plan.bn == 192 || tl_plan.bn == 256) w.bn = tl_plan.bn;  // tuned or loaded
  const int64_t tiles = cdiv(g->co, BM) * cdiv(w.vchunks, w.bn / 32);
  const int per_tile = w.bn / 32;
  // CTA pairs: two co tiles share the x columns, each CTA staging half of them (full tiles only, not the window mode)
  // (measured at batch 256: 256-column tiles +5..16 %, e.g. 256 -> 256 3x3 at 14^2 0.310 -> 0.271 ms; 128-column tiles lose a
  // third, their stages being too short to hide the cross-SM barrier round trip)
  w.pair = !window && !paired_taps && w.bn >= 192 && cdiv(g->co, BM) % 2 == 0 && w.chunks % per_tile == 0 && per_tile % 2 == 0 && g->co % 32 == 0 &&
           g->ci % 32 == 0 && cta_pairs_enabled();
  const int per_cta = w.pair ? per_tile / 2 : per_tile;
  w.cpi = std::gcd(w.cblocks, per_cta);  // 32-channel blocks one x box carries: a box never straddles two taps, two tiles or two CTAs
  const bool aligned_taps = true;
  const bool matrix = !window && g->ks == 1 && g->stride == 1 && g->pad == 0 && g->ci % 32 == 0;
  const bool rect = !window && !matrix && g->ci % 32 == 0 && g->co % 32 == 0 && aligned_taps && g->stride <= 8;
  // x boxes per stage: 1 in matrix mode, per_tile / cpi in rectangle mode, per_tile in window / im2col mode
  const bool few_boxes = (matrix && g->co % 32 == 0) || (rect && per_cta / w.cpi <= 2);
  // 16-pixel stages (twice as many of them) only where 32-pixel ones would leave a ring of two: wide single-CTA tiles whose x
  // operand is one box. Elsewhere a stage's barrier hand-offs cost more than the deeper ring gains (measured at batch 256:
  // 64 -> 256 1x1 0.324 -> 0.269 ms, 128 -> 128 3x3 0.398 -> 0.332 with 32-pixel stages; 256 -> 64 1x1 0.261 -> 0.288 the other way).
  const int PB = few_boxes && matrix && w.bn >= 192 && !w.pair ? 16 : 32;  // (a pair synchronises two SMs per stage: fewer, larger stages)
  w.pb = PB;
  int64_t total_blocks = cdiv((int64_t)g->n * g->oh * g->ow, PB);
  if (window) {
    w.mode = paired_rows ? 4 | 8 | 16 : 4 | 8;
    w.bw = PB; w.bh = 1; w.bn_img = 1;
  } else if (matrix) {
    w.mode = 2 | (g->co % 32 == 0 ? 1 : 0);
  } else if (rect) {
    // PB-pixel rectangles bw x bh x bn (powers of two) that waste the fewest pixels; wider rows on ties
    w.mode = paired_taps ? 4 | 16 : 4;
    double best = -1;
    for (int bw = PB; bw >= 1; bw >>= 1)
      for (int bh = PB / bw; bh >= 1; bh >>= 1) {
        const int bn = PB / (bw * bh);
        if (bw * g->stride > 256 || bh * g->stride > 256) continue;
        const double eff = ((double)g->ow * g->oh * g->n) /
                           ((double)cdiv(g->ow, bw) * bw * cdiv(g->oh, bh) * bh * cdiv(g->n, bn) * bn);
        if (eff > best + 1e-9) { best = eff; w.bw = bw; w.bh = bh; w.bn_img = bn; }
      }
  } else {
    w.mode = g->co % 32 == 0 ? 1 : 0;
  }
  if (w.mode & 4) {
    w.tiles_x = (int)cdiv(g->ow, w.bw); w.tiles_y = (int)cdiv(g->oh + w.shift_y, w.bh);  // (a row shift: blocks from row -1)
    total_blocks = (int64_t)w.tiles_x * w.tiles_y * cdiv(g->n, w.bn_img);
  }
  w.total_blocks = (int)total_blocks;
  // one wave of CTAs: a CTA's fixed cost (TMEM allocation, first loads, 128 KB partial tile written and summed later) is
  // worth 5-10 k-blocks, so fewer and longer split-K slices win over finer load balance (measured with 1-4 waves)
  int64_t want = std::max<int64_t>(1, sm_count() / tiles);
  if (tl_plan.mult > 0) want = std::max<int64_t>(1, (int64_t)(want * tl_plan.mult + 0.5));
  const int64_t slices = std::max<int64_t>(1, std::min<int64_t>(want, total_blocks / 8));
  w.blocks_per_slice = (int)cdiv(total_blocks, slices);
  w.slices = (int)cdiv(total_blocks, w.blocks_per_slice);
  w.part_floats = (size_t)w.slices * g->co * w.chunks * 32;
  return w;
}

#define OMT_ENCODE(call, what)                                   \
  do {                                                           \
    CUresult r_ = (call);                                        \
    if (r_ != CUDA_SUCCESS) {                                    \
      set_error("%s failed (%d)", what, (int)r_);                \
      return OMT_ECUDA;                                          \
    }                                                            \
  } while (0)

// `x` is the channels-last activation, or in window mode the padded 4-channel staging copy
template <int BN, int PB, bool PAIR = false>
int launch_wgrad(const OmtConvGeo* g, const WgPlan& w, const float* x, const float* gy, float* part, cudaStream_t s) {
  using S = WgSmem<BN, PB, PAIR>;
  alignas(64) CUtensorMap map_x, map_g;
  const int64_t P = (int64_t)g->n * g->oh * g->ow;
  constexpr auto F32 = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  constexpr auto SW = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
  constexpr auto IL = CU_TENSOR_MAP_INTERLEAVE_NONE;
  constexpr auto L2P = CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  constexpr auto FILL = CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE;
  // ---- x ----
  if (w.mode & 8) {
    // staging copy [n][ih][ws][4]: dims (floats of a window row, ox with overlapping stride, input row, image)
    const WinPlan wp = plan_window(g);
    cuuint64_t dims[4] = {(cuuint64_t)wp.kb * BKF, (cuuint64_t)g->ow, (cuuint64_t)g->ih, (cuuint64_t)g->n};
    cuuint64_t strides[3] = {(cuuint64_t)g->stride * 16, (cuuint64_t)wp.ws * 16, (cuuint64_t)g->ih * wp.ws * 16};
    cuuint32_t box[4] = {BKF, PB, 1, 1}, estr[4] = {1, 1, 1, 1};
    OMT_ENCODE(g_encode_tiled(&map_x, F32, 4, (void*)x, dims, strides, box, estr, IL, SW, L2P, FILL), "cuTensorMapEncodeTiled (window rows)");
  } else if (w.mode & 4) {
    cuuint64_t dims[5] = {32, (cuuint64_t)g->iw, (cuuint64_t)g->ih, (cuuint64_t)g->n, (cuuint64_t)(g->ci / 32)};
    cuuint64_t strides[4] = {(cuuint64_t)g->ci * 4, (cuuint64_t)g->iw * g->ci * 4, (cuuint64_t)g->ih * g->iw * g->ci * 4, 128};
    cuuint32_t box[5] = {BKF, (cuuint32_t)(w.bw * g->stride), (cuuint32_t)(w.bh * g->stride), (cuuint32_t)w.bn_img, (cuuint32_t)w.cpi};
    cuuint32_t estr[5] = {1, (cuuint32_t)g->stride, (cuuint32_t)g->stride, 1, 1};
    OMT_ENCODE(g_encode_tiled(&map_x, F32, 5, (void*)x, dims, strides, box, estr, IL, SW, L2P, FILL), "cuTensorMapEncodeTiled (x rectangles)");
  } else if (w.mode & 2) {
    // x is the row-major [P, ci] matrix: dims (32 channels, pixel, 32-channel block), one box = the whole B tile
    cuuint64_t dims[3] = {32, (cuuint64_t)P, (cuuint64_t)(g->ci / 32)};
    cuuint64_t strides[2] = {(cuuint64_t)g->ci * 4, 128};
    cuuint32_t box[3] = {BKF, PB, (cuuint32_t)S::B_CHUNKS}, estr[3] = {1, 1, 1};
    OMT_ENCODE(g_encode_tiled(&map_x, F32, 3, (void*)x, dims, strides, box, estr, IL, SW, L2P, FILL), "cuTensorMapEncodeTiled (x matrix)");
  } else {
    cuuint64_t dims[4] = {(cuuint64_t)g->ci, (cuuint64_t)g->iw, (cuuint64_t)g->ih, (cuuint64_t)g->n};
    cuuint64_t strides[3] = {(cuuint64_t)g->ci * 4, (cuuint64_t)g->iw * g->ci * 4, (cuuint64_t)g->ih * g->iw * g->ci * 4};
    int lower[2] = {-g->pad, -g->pad}, upper[2] = {g->pad - (g->ks - 1), g->pad - (g->ks - 1)};
    cuuint32_t estr[4] = {1, (cuuint32_t)g->stride, (cuuint32_t)g->stride, 1};
    OMT_ENCODE(g_encode_im2col(&map_x, F32, 4, (void*)x, dims, strides, lower, upper, BKF, PB, estr, IL, SW, L2P, FILL), "cuTensorMapEncodeIm2col");
  }
  // ---- gy ----
  if (w.mode & 4) {
    cuuint64_t dims[5] = {32, (cuuint64_t)g->ow, (cuuint64_t)g->oh, (cuuint64_t)g->n, (cuuint64_t)(g->co / 32)};
    cuuint64_t strides[4] = {(cuuint64_t)g->co * 4, (cuuint64_t)g->ow * g->co * 4, (cuuint64_t)g->oh * g->ow * g->co * 4, 128};
    cuuint32_t box[5] = {BKF, (cuuint32_t)w.bw, (cuuint32_t)w.bh, (cuuint32_t)w.bn_img, (w.mode & 16) ? 2u : 4u}, estr[5] = {1, 1, 1, 1, 1};
    OMT_ENCODE(g_encode_tiled(&map_g, F32, 5, (void*)gy, dims, strides, box, estr, IL, SW, L2P, FILL), "cuTensorMapEncodeTiled (gy rectangles)");
  } else if (w.mode & 1) {  // gy [P, co]: the 128-channel tile as one box of four 32-channel blocks
    cuuint64_t dims[3] = {32, (cuuint64_t)P, (cuuint64_t)(g->co / 32)};
    cuuint64_t strides[2] = {(cuuint64_t)g->co * 4, 128};
    cuuint32_t box[3] = {BKF, PB, 4}, estr[3] = {1, 1, 1};
    OMT_ENCODE(g_encode_tiled(&map_g, F32, 3, (void*)gy, dims, strides, box, estr, IL, SW, L2P, FILL), "cuTensorMapEncodeTiled (gy blocks)");
  } else {
    cuuint64_t dims[2] = {(cuuint64_t)g->co, (cuuint64_t)P};
    cuuint64_t strides[1] = {(cuuint64_t)g->co * 4};
    cuuint32_t box[2] = {BKF, PB}, estr[2] = {1, 1};
    OMT_ENCODE(g_encode_tiled(&map_g, F32, 2, (void*)gy, dims, strides, box, estr, IL, SW, L2P, FILL), "cuTensorMapEncodeTiled (gy)");
  }
  static std::once_flag attr_once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(attr_once, [] { attr_err = cudaFuncSetAttribute((wgrad_tc_kernel<BN, PB, PAIR>), cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL); });
  OMT_CUDA(attr_err);
  WgArgs a{};
  a.mode = w.mode; a.total_blocks = w.total_blocks;
  a.bw = w.bw; a.bh = w.bh; a.bn = w.bn_img; a.tiles_x = w.tiles_x; a.tiles_y = w.tiles_y; a.cpi = w.cpi;
  a.part = part; a.P = g->n * g->oh * g->ow; a.co = g->co; a.oh = g->oh; a.ow = g->ow; a.ks = g->ks; a.stride = g->stride; a.pad = g->pad;
  a.cblocks = w.cblocks; a.cpad = w.cpad; a.chunks = w.vchunks; a.out_chunks = w.chunks;
  memcpy(a.top, w.top, sizeof(a.top)); memcpy(a.bot, w.bot, sizeof(a.bot)); a.shift_x = w.shift_x; a.shift_y = w.shift_y; a.blocks_per_slice = w.blocks_per_slice;
  dim3 grid((unsigned)cdiv(g->co, BM), (unsigned)cdiv(w.vchunks, BN / 32), (unsigned)w.slices);
  if constexpr (PAIR) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = dim3(WG_THREADS); cfg.dynamicSmemBytes = S::TOTAL; cfg.stream = s;
    cudaLaunchAttribute at{};
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at; cfg.numAttrs = 1;
    OMT_CUDA(cudaLaunchKernelEx(&cfg, wgrad_tc_kernel<BN, PB, true>, map_x, map_g, a));
    return check_launch(BN == 64 ? "wgrad_tc_256x64_pair" : (BN == 128 ? "wgrad_tc_256x128_pair" : (BN == 192 ? "wgrad_tc_256x192_pair" : "wgrad_tc_256x256_pair")));
  }
  wgrad_tc_kernel<BN, PB><<<grid, WG_THREADS, S::TOTAL, s>>>(map_x, map_g, a);
  if (w.mode & 16) return check_launch(BN == 64 ? "wgrad_tc_128x64_tap_pairs" : (BN == 128 ? "wgrad_tc_128x128_tap_pairs" : (BN == 192 ? "wgrad_tc_128x192_tap_pairs" : "wgrad_tc_128x256_tap_pairs")));
  return check_launch(BN == 64 ? "wgrad_tc_128x64" : (BN == 128 ? "wgrad_tc_128x128" : (BN == 192 ? "wgrad_tc_128x192" : "wgrad_tc_128x256")));
}

bool cl_ok(const OmtAct* a, int c, int h, int w) {
  return a && a->p && is_nhwc(a, c, h, w) && c % 4 == 0 && (reinterpret_cast<uintptr_t>(a->p) & 15) == 0;
}

}  // namespace

int tc_error_word() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

// kind 0: a = x, b = y.  kind 1: a = gy, b = dx.  kind 2: weight gradient (not on this path yet)
bool tc_supported(int kind, const OmtConvGeo* g, const OmtAct* a, const OmtAct* b) {
  if (!b || !b->p) return false;
  if (kind == 0) return (cl_ok(a, g->ci, g->ih, g->iw) && g->ci >= 8 && g->co >= 8 && g->pad < g->ks) || (a && a->p && window_ok(g));
  if (kind == 1) return cl_ok(a, g->co, g->oh, g->ow) && g->co >= 8 && g->ci >= 8 && g->pad < g->ks;
  // kind 2: a = x, b = gy
  if (!cl_ok(b, g->co, g->oh, g->ow) || g->co < 8 || g->pad >= g->ks) return false;
  if (g->ci <= 4) return a && a->p && window_ok(g) && g->co % 32 == 0;  // window mode reads x through a staging copy: any layout
  return cl_ok(a, g->ci, g->ih, g->iw) && g->ci >= 8;
}
// the stride-phase sub-convolutions of an input gradient, in launch order (csrc/conv.cpp:78-95 of the reference)
struct Phase { TcProblem p; int ky0, kx0, jy, jx; };
static std::vector<Phase> dgrad_phases(const OmtConvGeo* g, const float* gy) {
  std::vector<Phase> out;
  const int s = g->stride;
  for (int py = 0; py < s; py++)
    for (int px = 0; px < s; px++) {
      const int hi = (int)cdiv(g->ih - py, s), wi = (int)cdiv(g->iw - px, s);
      if (hi <= 0 || wi <= 0) continue;
      const int ky0 = (py + g->pad) % s, kx0 = (px + g->pad) % s;
      const int jy = ky0 < g->ks ? (int)cdiv(g->ks - ky0, s) : 0, jx = kx0 < g->ks ? (int)cdiv(g->ks - kx0, s) : 0;
      if (jy == 0 || jx == 0) continue;
      const int qy = (py + g->pad - ky0) / s, qx = (px + g->pad - kx0) / s;
      // output (i, j) of the phase reads gy[i + qy - ty, j + qx - tx]; with flipped taps ty' = jy-1-ty the first tap sits at qy-(jy-1)
      TcProblem p{gy, g->n, g->co, g->oh, g->ow, hi, wi, g->ci, jy, jx, 1, qy - (jy - 1), qx - (jx - 1), s, py, px};
      out.push_back({p, ky0, kx0, jy, jx});
    }
  return out;
}
static size_t dgrad_part_floats(const OmtConvGeo* g) {
  size_t m = 0;
  for (const Phase& ph : dgrad_phases(g, nullptr)) m = std::max(m, part_floats(ph.p));
  return m;
}

size_t tc_workspace(int kind, const OmtConvGeo* g) {
  if (kind == 0) {
    if (g->ci <= 4 && window_ok(g)) {
      WinPlan w = plan_window(g);
      return (((w.stage_floats + 63) / 64) * 64 + w.split_floats_) * sizeof(float) + 256;
    }
    TcProblem p{nullptr, g->n, g->ci, g->ih, g->iw, g->oh, g->ow, g->co, g->ks, g->ks, g->stride, -g->pad, -g->pad, 1, 0, 0};
    return (split_floats(g->co, g->ks, g->ci) + part_floats(p)) * sizeof(float) + 512;
  }
  if (kind == 1) return (split_floats(g->ci, g->ks, g->co) + dgrad_part_floats(g)) * sizeof(float) + 512;
  const WgPlan w = plan_wgrad(g);
  return (w.stage_floats + w.part_floats) * sizeof(float) + 256;
}

int tc_conv_fwd(const OmtConvGeo* g, const OmtAct* x, const float* w, const float* bias, const OmtAct* y, float* stats, uint32_t flags, void* ws,
                cudaStream_t s) {
  if (!load_driver_entry_points()) {
    set_error("the CUDA driver does not export cuTensorMapEncodeTiled/Im2col");
    return OMT_ECUDA;
  }
  if (g->ci <= 4) return run_window_fwd(g, x, w, bias, y, stats, flags, ws, s);
  TcProblem p{x->p, g->n, g->ci, g->ih, g->iw, g->oh, g->ow, g->co, g->ks, g->ks, g->stride, -g->pad, -g->pad, 1, 0, 0};
  SplitArgs sp{g->co, g->ci, g->ks, 0, 0, 0, 0, 0, 0, 1};
  float* part = (float*)ws + ((split_floats(g->co, g->ks, g->ci) + 63) / 64) * 64;
  return run_tc(p, w, sp, (float*)ws, part, y, bias, stats, flags, s);
}

// 32-row groups the forward kernel reports statistics for (0: this call cannot: not a tensor-core geometry, an output that
// is not dense channels-last, or a reduction split over CTAs). Same decisions as tc_conv_fwd makes.
int tc_bnstats_groups(const OmtConvGeo* g, const OmtAct* x, const OmtAct* y) {
  if (!tc_supported(0, g, x, y) || !is_nhwc(y, g->co, g->oh, g->ow) || g->co % 4 != 0 || (reinterpret_cast<uintptr_t>(y->p) & 15)) return 0;
  if (g->ci <= 4) {
    const WinPlan wp = plan_window(g);
    return g->n * wp.tiles_x * wp.tiles_y * 4;
  }
  TcProblem p{x->p, g->n, g->ci, g->ih, g->iw, g->oh, g->ow, g->co, g->ks, g->ks, g->stride, -g->pad, -g->pad, 1, 0, 0};
  const int64_t M = (int64_t)g->n * g->oh * g->ow;
  const int kblocks = g->ks * g->ks * (int)cdiv(g->ci, BKF);
  // With a short reduction a tile's time is its epilogue (the layer is bound by storing y) and the statistics lengthen
  // exactly that: on ResNet-50 at batch 256 they then cost more than the separate 4-byte-per-element pass over y they save
  // (measured per layer and in the whole step). Small problems are bound by launches instead, and there one launch less wins.
  if (kblocks < BNSTATS_MIN_KBLOCKS && M * g->co > BNSTATS_SMALL_OUTPUT) return 0;
  if (plan_splits(M, g->co, kblocks, pick_bn(p)) > 1) return 0;
  return (int)cdiv(M, BM) * 4;
}

// Input gradient as forward convolutions of gy. Stride 1: one convolution with the weights transposed and flipped and
// padding ks-1-pad. Stride s: one stride-1 convolution per phase (py, px) of the input grid, over the taps ky = ky0 + s*ty
// that reach that phase (the index algebra of the reference's host loop, csrc/conv.cpp:78-95), written to every s-th pixel;
// phases no tap reaches stay zero.
int tc_conv_dgrad(const OmtConvGeo* g, const OmtAct* gy, const float* w, const OmtAct* dx, uint32_t flags, void* ws, cudaStream_t st_) {
  const uint32_t epi = flags & OMT_EPI_ACCUM;
  if (!load_driver_entry_points()) {
    set_error("the CUDA driver does not export cuTensorMapEncodeTiled/Im2col");
    return OMT_ECUDA;
  }
  const int s = g->stride;
  float* wsplit = (float*)ws;
  float* part = (float*)ws + ((split_floats(g->ci, g->ks, g->co) + 63) / 64) * 64;  // shared by the phases: they run in order
  bool zeroed = false;
  for (int py = 0; py < s; py++)
    for (int px = 0; px < s; px++) {
      const int hi = (int)cdiv(g->ih - py, s), wi = (int)cdiv(g->iw - px, s);
      if (hi <= 0 || wi <= 0) continue;
      const int ky0 = (py + g->pad) % s, kx0 = (px + g->pad) % s;
      const int jy = ky0 < g->ks ? (int)cdiv(g->ks - ky0, s) : 0, jx = kx0 < g->ks ? (int)cdiv(g->ks - kx0, s) : 0;
      if (jy == 0 || jx == 0) {  // no tap lands on this phase: its pixels are zero (nothing to add when accumulating)
        if (!zeroed && !epi) {
          OMT_REQUIRE(is_nhwc(dx, g->ci, g->ih, g->iw) || is_nchw(dx, g->ci, g->ih, g->iw), "strided input gradient needs a dense dx");
          OMT_CUDA(cudaMemsetAsync(dx->p, 0, (size_t)g->n * g->ci * g->ih * g->iw * sizeof(float), st_));
          zeroed = true;
        }
        continue;
      }
    }
  for (int py = 0; py < s; py++)
    for (int px = 0; px < s; px++) {
      const int hi = (int)cdiv(g->ih - py, s), wi = (int)cdiv(g->iw - px, s);
      if (hi <= 0 || wi <= 0) continue;
      const int ky0 = (py + g->pad) % s, kx0 = (px + g->pad) % s;
      const int jy = ky0 < g->ks ? (int)cdiv(g->ks - ky0, s) : 0, jx = kx0 < g->ks ? (int)cdiv(g->ks - kx0, s) : 0;
      if (jy == 0 || jx == 0) continue;
      const int qy = (py + g->pad - ky0) / s, qx = (px + g->pad - kx0) / s;
      // output (i, j) of the phase reads gy[i + qy - ty, j + qx - tx]; with flipped taps ty' = jy-1-ty the first tap sits at qy-(jy-1)
      TcProblem p{gy->p, g->n, g->co, g->oh, g->ow, hi, wi, g->ci, jy, jx, 1, qy - (jy - 1), qx - (jx - 1), s, py, px};
      SplitArgs sp{g->co, g->ci, g->ks, 0, 0, 0, 1, ky0, kx0, s};
      int r = run_tc(p, w, sp, wsplit, part, dx, nullptr, nullptr, epi, st_);
      if (r) return r;
      wsplit += 2 * (size_t)g->ci * jy * jx * (cdiv(g->co, BKF) * BKF);
    }
  return OMT_OK;
}
int tc_conv_wgrad(const OmtConvGeo* g, const OmtAct* x, const OmtAct* gy, float* dw, float scale, void* ws, cudaStream_t s) {
  if (!load_driver_entry_points()) {
    set_error("the CUDA driver does not export cuTensorMapEncodeTiled/Im2col");
    return OMT_ECUDA;
  }
  const WgPlan w = plan_wgrad(g);
  float* part = (float*)ws + w.stage_floats;
  const float* xin = x->p;
  if (w.mode & 8) {  // padded 4-channel copy of x, as in the forward window mode
    const WinPlan wp = plan_window(g);
    const int64_t total = (int64_t)g->n * g->ih * wp.ws;
    stage_window_kernel<<<(unsigned)cdiv(total, 256), 256, 0, s>>>(view(x), (float*)ws, g->n, g->ci, g->ih, g->iw, wp.ws, g->pad);
    int r0 = check_launch("conv_tc_stage_window");
    if (r0) return r0;
    xin = (const float*)ws;
  }
  int r;
  switch (w.bn) {
#define OMT_WG(BN_)                                                                                                                   \
  (w.pair ? (w.pb == 16 ? launch_wgrad<BN_, 16, true>(g, w, xin, gy->p, part, s) : launch_wgrad<BN_, 32, true>(g, w, xin, gy->p, part, s)) \
          : (w.pb == 16 ? launch_wgrad<BN_, 16>(g, w, xin, gy->p, part, s) : launch_wgrad<BN_, 32>(g, w, xin, gy->p, part, s)))
    case 64: r = OMT_WG(64); break;
    case 128: r = OMT_WG(128); break;
    case 192: r = OMT_WG(192); break;
    default: r = OMT_WG(256); break;
#undef OMT_WG
  }
  if (r) return r;
  launch_wgrad_reduce(part, dw, g->co, g->ci, g->ks * g->ks, w.cpad, w.slices, scale, (w.mode & 8) ? g->ks : 0, w.win_kb, s);
  return check_launch("wgrad_tc_reduce");
}

}  // namespace omt
