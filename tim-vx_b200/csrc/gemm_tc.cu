// int8 GEMM / implicit-GEMM convolution with fused requantization on Blackwell
// tensor cores (sm_100a).
//
//   D[m][oc] = requant( sum_k A[m][k] * B[oc][k] + bias_full[oc] )
//
// A: activations, u8 or s8, K-contiguous: either a matrix [M][Kp] (a
//    channels-last tensor seen as pixels x channels, or an im2col matrix), or —
//    convolution mode — the channels-last input itself as a 4-D tensor
//    (C, W, H, N), one filter tap per k-block fetched as a shifted TMA box, or
//    — halo mode, stride 1 with resident weights — the tile's input patch
//    fetched once per channel block and every tap an MMA on a shifted view of
//    it (GemmParams::halo).
// B: weights shifted into int8, [Np][Kp] K-contiguous.
// Both are "K-major" operands, which is what TMA tiled loads with a 32/64/128
// byte swizzle and tcgen05.mma.kind::i8 consume directly; accumulation is int32
// in tensor memory (TMEM).
//
// One persistent CTA per SM, 640 threads, warp-specialised:
//   warp 0      A producer   per stage: wait slot free, expect_tx, one TMA box
//   warp 2      B producer   per k-block (lanes issue the boxes of a stage in
//                            one instruction).  Two warps because a single
//                            thread's wait/expect/issue sequence, not memory,
//                            bounded the load rate.
//   warp 1      MMA issuer   allocates TMEM; one lane issues M=128,N=BN,K=32
//                            MMAs and commits them to mbarriers: slot-free
//                            after each stage, accumulator-ready after a tile.
//   warps 4-19  epilogue     16 warps (four per SM scheduler, to hide latency).
//                            A warp owns the 32 TMEM lanes (tile rows) its id
//                            maps to and every fourth 16-column chunk:
//                            tcgen05.ld (the next chunk's load in flight),
//                            folded bias, requantize two floats per
//                            instruction, saturating pack, and a 16-byte store
//                            per thread straight to the output.  No barrier
//                            joins the warps, so they drift apart and work on
//                            neighbouring tiles; two accumulator buffers
//                            overlap tile i's epilogue with tile i+1's MMAs.
//                            (B2VX_TC_STORE=tma: write the bytes swizzled into
//                            a staging tile instead and store it with TMA.)
//                            Tiles of at most 64 columns: four teams of four
//                            warps, each team on its own tile with all chunks.
//   warp 3      residual producer of a fused Add (template FUSE): the Add's
//                            64 KB table by four bulk copies first, then the
//                            Add's other operand, tile by tile, into the
//                            staging memory by TMA; the epilogue looks every
//                            (own byte, residual byte) pair up in the table.
// Small weight tiles (BN x K up to 72 KB) are loaded once by warp 2 and stay in
// shared memory; the ring then holds A only.  Long K loops with many tiles per
// CTA run two M tiles at once on one stream of weight blocks (GemmParams::pair).
// A stage holds up to `group` k-blocks so that small k-blocks share one
// barrier round trip.  The grid is a multiple of the number of N tiles: a CTA
// keeps one N tile for life (bias and scales staged in shared memory once) and
// neighbouring CTAs share an A row-block, whose repeated reads hit L2.
//
// Every mbarrier wait is bounded: after kWaitLimitCycles the waiting thread
// records a code in *status, raises a CTA-wide abort flag that all other waits
// poll, and the CTA falls through to its common exit where outstanding TMA
// stores are drained and tensor memory is released.  Every CTA is on its own:
// no cluster launch, every load has exactly one destination CTA.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "kernels.h"
#include "pdl.cuh"
#include "requant.cuh"

// Build with -DB2VX_TC_TRACE to record, for CTA 0, when each role passed its waits (a debugging aid
// for pipeline stalls; the normal build contains none of it).  -DB2VX_TRACE_WARP=<4..19> picks the epilogue
// warp whose per-tile stamps (loop top, accumulator ready, residual ready, chunks done) are printed.
// -DB2VX_ABL_NOREQ / -DB2VX_ABL_NOLUT build an epilogue without its requantization / without the fused Add's
// table look-ups: wrong outputs, for measuring what each part costs.
#ifdef B2VX_TC_TRACE
#define TC_TRACE(role, idx, slot) \
  do { if (p.trace && blockIdx.x == 0 && (idx) < 64) p.trace[((role) * 64 + (idx)) * 2 + (slot)] = clock64(); } while (0)
#define TC_MARK(k) \
  do { if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) p.trace[384 + (k)] = clock64(); } while (0)
#ifndef B2VX_TRACE_WARP
#define B2VX_TRACE_WARP 4
#endif
#define TC_EPI(j, k) \
  do { if (p.trace && blockIdx.x == 0 && threadIdx.x == B2VX_TRACE_WARP * 32 && (j) < 16) p.trace[400 + (j) * 8 + (k)] = clock64(); } while (0)
#else
#define TC_TRACE(role, idx, slot) do { } while (0)
#define TC_MARK(k) do { } while (0)
#define TC_EPI(j, k) do { } while (0)
#endif

namespace b2vx {

namespace {

constexpr int kBlockM = 128;
constexpr int kFirstEpilogueWarp = 4;
#ifndef B2VX_EPI_WARPS
#define B2VX_EPI_WARPS 16
#endif
constexpr int kEpilogueWarps = B2VX_EPI_WARPS;   // a multiple of four: one warp per TMEM lane quarter in every column group
constexpr int kGroups = kEpilogueWarps / 4;      // column groups of a wide tile, or teams on narrow tiles
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kThreadsTc = (kFirstEpilogueWarp + kEpilogueWarps) * 32;
constexpr int kMaxStages = 8;
constexpr int kMaxGroup = 8;
constexpr int kMaxAccBuffers = 8;
constexpr long long kWaitLimitCycles = 2000000000LL;  // about one second
constexpr int kSmemBudget = 226 * 1024;               // dynamic shared memory requested at most
constexpr int kMinDynSmem = 120 * 1024;               // keeps two CTAs from sharing an SM (and its TMEM)

struct GemmParams {
  int M, Ocp, ldd;
  int BN, BK, n_tiles, m_tiles, num_kb, stages;   // BN: MMA N = weight rows per N tile
  int BNd;                 // output channels per N tile (BN, or BN - 16 when the tile carries the ones row)
  int group;               // k-blocks per pipeline stage
  int tmem_cols;
  int acc_stride;          // TMEM columns between accumulator buffers (BN rounded up to 32)
  int acc_shift;           // log2 of the number of accumulator buffers (2, 4 or 8 of them)
  // Narrow tiles (at most four 16-column chunks): the sixteen epilogue warps split into four teams of four
  // (one warp per TMEM lane quarter), each team takes every fourth tile of the CTA and all of its chunks, so
  // that a warp's per-tile work (waits, row arithmetic) is spread over four chunks as it is with wide tiles.
  int teams;
  // The CTA's weight tile (all k-blocks of its N tile) stays in shared memory for the whole kernel, loaded once
  // before the first tile; the ring then carries the A operand only.  For narrow layers, which are bound
  // by the operand traffic from L2, this removes a third to two thirds of it.
  int b_resident;
  uint32_t idesc;
  uint32_t layout_type;    // UMMA smem descriptor swizzle code
  uint32_t sbo;            // bytes between 8-row groups
  ContractEpilogue ep;
  uint8_t* D;
  int* status;
  // implicit-GEMM convolution (conv != 0): one M tile is TW x TH x TN output pixels and one k-block is
  // (filter tap, channel block).
  int conv;
  int TW, TH, TN, tiles_w, tiles_h;
  int Wo, Ho, Nimg;
  int kw, sx, sy, dx, dy, pl, pt;
  int cblocks, Cp;
  uint32_t a_tx_bytes;     // bytes one A box delivers (rows in the box x BK)
  // Halo mode of the implicit convolution (stride 1, weights resident): the ring's stage is the tile's input patch
  // with its halo for one channel block, loaded once ((TW + kw - 1) x (TH + kh - 1) pixels of BK bytes, TW = 8,
  // TN = 1), and the kh * kw taps are MMAs on shifted views of it: descriptor start = patch + (ky * halo_w + kx) * BK,
  // distance between 8-row groups = halo_w * BK.  The 64-byte swizzle is a function of the absolute shared-memory
  // address on both sides (TMA write, MMA read), so a view may start on any pixel.
  int halo, halo_w, halo_kh;   // halo_kh: filter rows (kept here so that the issuing thread does not divide)
  uint32_t a_stage_bytes;  // halo mode: bytes of a stage (the patch, rounded up to 1 KB)
  int num_kb_b;            // k-blocks of the weight tile (kh * kw * cblocks; == num_kb unless halo)
  // Pair mode (plain GEMM with a long K loop): a CTA works on two of its M tiles at once, one per accumulator buffer,
  // and every stage holds [A of the first | A of the second | B], so the weight block is fetched once for 256 rows:
  // 64 instead of 96 bytes per 128 x 256 x 128 block of multiply-accumulates, which the SM's read port from L2
  // (about 56 bytes per clock) could not feed.  The price: both accumulators are in use, so a pair's epilogue does
  // not overlap the next pair's main loop; chosen only where the main loop is many times longer.
  int pair;
  // output through shared memory + TMA store: the tile is staged as BN/store_span column blocks of
  // [128 rows][store_span bytes], 16-byte chunks XOR-swizzled the way the store's tensor map expects.
  // store_span == 0: BN is not a multiple of 32, threads store their 16-byte pieces directly.
  int store_span;
  // FUSE: the residual tile comes into the same staging memory by TMA (tensor map in the output map's
  // slot, column blocks of res_span bytes); 0: BN is not a multiple of 32, threads load their pieces.
  int res_span;
  int dz;                  // weight zero point left after the shift into int8; != 0: column BNd of the accumulator is S
  int exact_only;          // requantize with the exact sequence only (the fast form's range check failed)
  long long wait_limit;    // cycles after which a barrier wait gives up (kWaitLimitCycles)
  uint32_t tx_extra;       // test aid: bytes added to what the A producer announces, so that its barrier never completes
#ifdef B2VX_TC_TRACE
  long long* trace;        // clock64 stamps of CTA 0, [3 roles][64 iterations][2], 16 marks, then [16 tiles][8] of one epilogue warp
#endif
};

// ---- PTX wrappers -----------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// try_wait may suspend the thread in hardware until the phase completes or the hint (ns) runs out,
// which keeps waiting warps out of the issue slots the epilogue warps need.
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(20000u)
      : "memory");
  return ok;
}

// Bounded wait.  Returns false when the CTA is aborting.  Polls back off: a wait that is not over after
// a few tries is a long one (a control warp waiting for the epilogue, say), and a warp that keeps
// polling takes issue slots from the warps it is waiting for; sleeps grow from 64 ns to 1 us.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          long long limit = kWaitLimitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  unsigned sleep_ns = 32;
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 4; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > limit) {
      *abort_flag = 1;
      atomicCAS(status, 0, code);
      return false;
    }
    if (sleep_ns < 1024) sleep_ns <<= 1;
    __nanosleep(sleep_ns);
  }
}

// One lane of a fully converged warp.  The control warps run their loops with all 32 lanes (so that
// every value feeding a TMA or MMA instruction is warp-uniform and can live in uniform registers)
// and elect a single lane only for the issue itself.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
// Plain (untiled) bulk copy global -> shared: both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's store groups still have to read their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Makes this thread's shared-memory writes visible to the TMA engine (async proxy).
__device__ __forceinline__ void fence_smem_to_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Barrier among the epilogue warps only.
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same with the accumulate flag known when compiling (no predicate set-up per instruction).
template <int ACCUMULATE>
__device__ __forceinline__ void tc_mma_i8_const(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "n"(ACCUMULATE)
      : "memory");
}

// The issue loops keep a descriptor as its two 32-bit halves: only the low half (start address in 16-byte units, bits
// 0-13) changes from one instruction to the next, by additions that never carry out of that field (shared-memory
// addresses stay below 256 KB), so advancing a descriptor is one 32-bit addition.
template <int ACCUMULATE>
__device__ __forceinline__ void tc_mma_i8_halves(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t}"
      ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "n"(ACCUMULATE)
      : "memory");
}

__device__ __forceinline__ void tc_ld_32x16(uint32_t taddr, int (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld_32x1(uint32_t taddr, int& r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_wait1(int& r) { asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r) : : "memory"); }
// The load is asynchronous: its destination registers are valid only after tcgen05.wait::ld.  The wait
// names them as read-write operands so that the compiler orders every use of them after it.
__device__ __forceinline__ void tc_ld_wait(int (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are one
// swizzle span wide: start address, LBO = 1 (unused for swizzled K-major),
// SBO = 8 rows, descriptor version 1, swizzle code in bits 61-63.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(layout_type & 7) << 61;
  return d;
}

struct SmemHeader {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long tmem_full[kMaxAccBuffers];
  unsigned long long tmem_empty[kMaxAccBuffers];
  unsigned long long b_full;         // resident weights landed
  unsigned long long tab_full;       // FUSE: the Add's table landed
  unsigned long long res_full[2];    // FUSE: residual tile landed / read by all epilogue warps
  unsigned long long res_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  // this CTA's N tile: folded bias and accumulator scale per column; read as 128-bit vectors
  alignas(16) int bias[256];
  alignas(16) float scale[256];
};

// EXTRA: rows carry a weight-zero-point term (p.dz, S column) and/or border corrections
// (p.ep.border_corr); the plain form contains no code for either.
// FUSE: a residual Add follows the convolution and is done here: the 64 KB table of that Add sits in
// shared memory behind the operand ring, the epilogue loads the residual's 16 bytes beside its own
// and stores the table's answers instead (direct stores only).
template <bool EXTRA, bool FUSE>
__global__ void __launch_bounds__(kThreadsTc, 1)
gemm_i8_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_d, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  TC_MARK(0);
  pdl_trigger();   // the next kernel of the stream may begin its own prologue
  // [ring of stages | two staging tiles | header], the first two 1024-byte aligned (128-byte swizzle)
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* tiles = smem_raw + (tiles_addr - raw_addr);
  const uint32_t a_bytes = p.halo ? p.a_stage_bytes : static_cast<uint32_t>(kBlockM) * p.BK;
  const uint32_t b_bytes = static_cast<uint32_t>(p.BN) * p.BK;
  const uint32_t sub_bytes = (p.pair ? 2u : 1u) * a_bytes + (p.b_resident ? 0u : b_bytes);   // one k-block: whole swizzle atoms, see the host-side plan
  const uint32_t b_off = (p.pair ? 2u : 1u) * a_bytes;   // B behind the A block(s) of a k-block
  const uint32_t stage_bytes = sub_bytes * p.group;
  const uint32_t ring_bytes = (p.stages * stage_bytes + 1023u) & ~1023u;
  const uint32_t bres_bytes = p.b_resident ? ((static_cast<uint32_t>(p.num_kb_b) * b_bytes + 1023u) & ~1023u) : 0u;
  const uint32_t bres_addr = tiles_addr + ring_bytes;                    // resident weights: k-block after k-block
  const uint32_t staging_bytes = (p.store_span || p.res_span) ? static_cast<uint32_t>(kBlockM) * p.BNd : 0u;   // per buffer, multiple of 4096
  uint8_t* staging = tiles + ring_bytes + bres_bytes;
  uint8_t* add_tab = staging + 2 * staging_bytes;                 // 64 KB when FUSE
  SmemHeader* hdr = reinterpret_cast<SmemHeader*>(add_tab + (FUSE ? 65536 : 0));
  volatile int* abort_flag = &hdr->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 32) {
    // descriptor fetches overlap the rest of the prologue instead of delaying the first loads
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
    if (p.store_span || p.res_span) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_d)) : "memory");
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&hdr->full[s]), p.b_resident ? 1 : 2);     // A producer (+ B producer)
      mbar_init(smem_u32(&hdr->empty[s]), 1);
    }
    for (int a = 0; a < kMaxAccBuffers; ++a) {
      mbar_init(smem_u32(&hdr->tmem_full[a]), 1);
      mbar_init(smem_u32(&hdr->tmem_empty[a]), p.teams ? 4 : kEpilogueWarps);
    }
    mbar_init(smem_u32(&hdr->b_full), 1);
    mbar_init(smem_u32(&hdr->tab_full), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&hdr->res_full[b]), 1);
      mbar_init(smem_u32(&hdr->res_empty[b]), kEpilogueWarps);
    }
    hdr->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const int n_tile = blockIdx.x % p.n_tiles;   // fixed per CTA: gridDim.x is a multiple of n_tiles
  // hence the j-th tile of this CTA is M tile m_tile0 + j * m_step (no division per tile)
  const int m_tile0 = blockIdx.x / p.n_tiles, m_step = gridDim.x / p.n_tiles;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&hdr->tmem_base)),
                 "r"(static_cast<uint32_t>(p.tmem_cols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = hdr->tmem_base;
  TC_MARK(1);

  if (warp == 2 && p.b_resident) {
    // ------------------------------------------------------------ resident weights: one load of every k-block
    // Weights are constants of the graph, so this does not wait for earlier kernels of the stream.
    if (elect_one()) {
      const uint32_t full = smem_u32(&hdr->b_full);
      mbar_arrive_expect_tx(full, static_cast<uint32_t>(p.num_kb_b) * b_bytes);
      int tap = 0, cb = 0;
      for (int kb = 0; kb < p.num_kb_b; ++kb) {
        const uint32_t dst = bres_addr + static_cast<uint32_t>(kb) * b_bytes;
        if (p.conv) {
          tma_load_2d(dst, &map_b, tap * p.Cp + cb * p.BK, n_tile * p.BN, full);
          if (++cb == p.cblocks) { cb = 0; ++tap; }
        } else {
          tma_load_2d(dst, &map_b, kb * p.BK, n_tile * p.BN, full);
        }
      }
    }
    __syncwarp();
  } else if (warp == 0 || warp == 2) {
    // ------------------------------------------------------------ TMA producers (warp 0: A, warp 2: B)
    // All lanes wait for the slot; one elected lane announces the bytes and issues the boxes of the
    // stage's k-blocks.
    const bool is_a = warp == 0;
    uint32_t it = 0, s = 0, ph = 0;   // stage index and ring phase, advanced without divisions
    // Everything above touched only constants and this CTA's own shared/tensor memory.  The operand
    // loads are the first access to what earlier kernels of the stream produced (and every later
    // access of this kernel, the output stores included, depends on them through the barriers).
    pdl_wait();
    bool ok = true;
    int m_tile = m_tile0;
    const int tstep = p.pair ? 2 : 1;   // pair mode: tiles j and j + 1 of this CTA go through the ring together
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += tstep * gridDim.x, m_tile += tstep * m_step) {
      const bool two = p.pair && tile + static_cast<int>(gridDim.x) < num_tiles;
      int w0 = 0, h0 = 0, n0 = 0;
      if (p.conv) {
        // tile -> first output pixel (tw, th, tn), turned into input coordinates of tap (0,0).
        // Coordinates left of / above the image are negative and read as zero (the padding).
        const int tw = m_tile % p.tiles_w, rest = m_tile / p.tiles_w;
        w0 = tw * p.TW * p.sx - p.pl;
        h0 = (rest % p.tiles_h) * p.TH * p.sy - p.pt;
        n0 = (rest / p.tiles_h) * p.TN;
      }
      int tap = 0, cb = 0, ky = 0, kx = 0;   // conv mode: k-block -> (tap = ky*kw + kx, channel block), stepped
      for (int kb0 = 0; kb0 < p.num_kb; kb0 += p.group, ++it) {
        const int cnt = min(p.group, p.num_kb - kb0);
        const uint32_t full = smem_u32(&hdr->full[s]);
        ok = mbar_wait(smem_u32(&hdr->empty[s]), ph ^ 1, abort_flag, p.status, is_a ? 1 : 5, p.wait_limit);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (is_a) TC_TRACE(0, it, 0);
        if (elect_one()) {
          mbar_arrive_expect_tx(full, static_cast<uint32_t>(cnt) * (is_a ? p.a_tx_bytes * (two ? 2u : 1u) : b_bytes) + (is_a ? p.tx_extra : 0u));
          uint32_t dst = tiles_addr + s * stage_bytes;
          int t_tap = tap, t_cb = cb, t_ky = ky, t_kx = kx;
          for (int gi = 0; gi < cnt; ++gi, dst += sub_bytes) {
            if (p.conv) {
              if (is_a) tma_load_4d(dst, &map_a, t_cb * p.BK, w0 + t_kx * p.dx, h0 + t_ky * p.dy, n0, full);
              else tma_load_2d(dst + b_off, &map_b, t_tap * p.Cp + t_cb * p.BK, n_tile * p.BN, full);
              if (++t_cb == p.cblocks) {
                t_cb = 0;
                ++t_tap;
                if (++t_kx == p.kw) { t_kx = 0; ++t_ky; }
              }
            } else if (is_a) {
              tma_load_2d(dst, &map_a, (kb0 + gi) * p.BK, m_tile * kBlockM, full);
              if (two) tma_load_2d(dst + a_bytes, &map_a, (kb0 + gi) * p.BK, (m_tile + m_step) * kBlockM, full);
            } else {
              tma_load_2d(dst + b_off, &map_b, (kb0 + gi) * p.BK, n_tile * p.BN, full);
            }
          }
        }
        __syncwarp();
        if (p.conv) {
          for (int gi = 0; gi < cnt; ++gi) {
            if (++cb == p.cblocks) {
              cb = 0;
              ++tap;
              if (++kx == p.kw) { kx = 0; ++ky; }
            }
          }
        }
        if (is_a) TC_TRACE(0, it, 1);
        if (++s == static_cast<uint32_t>(p.stages)) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    uint32_t it = 0, s = 0, ph = 0;
    bool ok = true;
    int j = 0;
    const int ksteps = p.BK >> 5;
    if (p.b_resident && static_cast<int>(blockIdx.x) < num_tiles) {
      ok = mbar_wait(smem_u32(&hdr->b_full), 0, abort_flag, p.status, 8, p.wait_limit);
      ok = __all_sync(0xffffffffu, ok);
    }
    const int tstep = p.pair ? 2 : 1;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += tstep * gridDim.x, j += tstep) {
      const uint32_t a = j & ((1 << p.acc_shift) - 1), aph = (j >> p.acc_shift) & 1;
      // pair mode (two accumulator buffers): tile j fills buffer 0 and tile j + 1, when the CTA has one, buffer 1
      const bool two = p.pair && tile + static_cast<int>(gridDim.x) < num_tiles;
      ok = mbar_wait(smem_u32(&hdr->tmem_empty[a]), aph ^ 1, abort_flag, p.status, 2, p.wait_limit);
      if (ok && two) ok = mbar_wait(smem_u32(&hdr->tmem_empty[a + 1]), aph ^ 1, abort_flag, p.status, 2, p.wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + a * p.acc_stride;
      uint32_t accumulate = 0;
      for (int kb0 = 0; kb0 < p.num_kb; kb0 += p.group, ++it) {
        ok = mbar_wait(smem_u32(&hdr->full[s]), ph, abort_flag, p.status, 3, p.wait_limit);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        TC_TRACE(1, it, 0);
        tc_fence_after();
        const int cnt = min(p.group, p.num_kb - kb0);
        if (p.halo) {
          // one stage = the input patch of channel block kb0: every tap is a shifted view of it.  The issuing thread
          // shares its scheduler with four epilogue warps, so every instruction here costs several cycles: descriptors
          // are built once per stage and advanced by additions to their address field (16-byte units).
          if (elect_one()) {
            const uint64_t da0 = make_smem_desc(tiles_addr + s * stage_bytes, static_cast<uint32_t>(p.halo_w) * p.BK, p.layout_type);
            const uint64_t db0 = make_smem_desc(bres_addr + static_cast<uint32_t>(kb0) * b_bytes, p.sbo, p.layout_type);
            const uint32_t a_hi = static_cast<uint32_t>(da0 >> 32), b_hi = static_cast<uint32_t>(db0 >> 32);
            uint32_t b_lo = static_cast<uint32_t>(db0);
            const uint32_t db_step = (static_cast<uint32_t>(p.cblocks) * b_bytes) >> 4;
            const uint32_t px16 = static_cast<uint32_t>(p.BK) >> 4;           // one pixel of the patch, in 16-byte units
            const int taps_h = p.halo_kh;
            bool first = accumulate == 0;
            if (p.kw == 3 && taps_h == 3) {
              // The 3x3 window written out (halo mode always has 64-byte channel blocks: a pixel is four 16-byte units,
              // two k steps): eighteen instructions whose descriptors differ by constants, no loop control between them.
              uint32_t a_row = static_cast<uint32_t>(da0);
              const uint32_t row16 = static_cast<uint32_t>(p.halo_w) * 4u;
#pragma unroll
              for (int ky = 0; ky < 3; ++ky, a_row += row16) {
#pragma unroll
                for (int kx = 0; kx < 3; ++kx, b_lo += db_step) {
                  const uint32_t a_lo = a_row + 4u * kx;
                  if (ky == 0 && kx == 0 && first) tc_mma_i8_halves<0>(tmem_d, a_lo, a_hi, b_lo, b_hi, p.idesc);
                  else tc_mma_i8_halves<1>(tmem_d, a_lo, a_hi, b_lo, b_hi, p.idesc);
                  tc_mma_i8_halves<1>(tmem_d, a_lo + 2u, a_hi, b_lo + 2u, b_hi, p.idesc);
                }
              }
            } else {
              for (int ky = 0; ky < taps_h; ++ky) {
                uint32_t a_lo = static_cast<uint32_t>(da0) + static_cast<uint32_t>(ky * p.halo_w) * px16;
                for (int kx = 0; kx < p.kw; ++kx, a_lo += px16, b_lo += db_step) {
                  if (first) {
                    tc_mma_i8_halves<0>(tmem_d, a_lo, a_hi, b_lo, b_hi, p.idesc);
                    first = false;
                  } else {
                    tc_mma_i8_halves<1>(tmem_d, a_lo, a_hi, b_lo, b_hi, p.idesc);
                  }
                  for (int k = 1; k < ksteps; ++k) tc_mma_i8_halves<1>(tmem_d, a_lo + 2u * k, a_hi, b_lo + 2u * k, b_hi, p.idesc);
                }
              }
            }
            tc_commit(smem_u32(&hdr->empty[s]));
          }
        } else if (elect_one()) {
          const uint64_t da0 = make_smem_desc(tiles_addr + s * stage_bytes, p.sbo, p.layout_type);
          const uint64_t db0 = make_smem_desc(p.b_resident ? bres_addr + static_cast<uint32_t>(kb0) * b_bytes : tiles_addr + s * stage_bytes + b_off,
                                              p.sbo, p.layout_type);
          const uint32_t a_hi = static_cast<uint32_t>(da0 >> 32), b_hi = static_cast<uint32_t>(db0 >> 32);
          uint32_t a_lo = static_cast<uint32_t>(da0), b_lo = static_cast<uint32_t>(db0);
          const uint32_t da_step = sub_bytes >> 4, db_step = (p.b_resident ? b_bytes : sub_bytes) >> 4;
          const uint32_t a2 = a_bytes >> 4;            // pair mode: the second tile's A block follows the first's
          const uint32_t tmem_d2 = tmem_d + p.acc_stride;
          bool first = accumulate == 0;
          if (two) {
            for (int gi = 0; gi < cnt; ++gi, a_lo += da_step, b_lo += db_step) {
              // k steps advance 32 bytes along K inside the swizzle span: +2 in 16-byte units
              if (first) {
                tc_mma_i8_halves<0>(tmem_d, a_lo, a_hi, b_lo, b_hi, p.idesc);
                tc_mma_i8_halves<0>(tmem_d2, a_lo + a2, a_hi, b_lo, b_hi, p.idesc);
                first = false;
              } else {
                tc_mma_i8_halves<1>(tmem_d, a_lo, a_hi, b_lo, b_hi, p.idesc);
                tc_mma_i8_halves<1>(tmem_d2, a_lo + a2, a_hi, b_lo, b_hi, p.idesc);
              }
              for (int k = 1; k < ksteps; ++k) {
                tc_mma_i8_halves<1>(tmem_d, a_lo + 2u * k, a_hi, b_lo + 2u * k, b_hi, p.idesc);
                tc_mma_i8_halves<1>(tmem_d2, a_lo + a2 + 2u * k, a_hi, b_lo + 2u * k, b_hi, p.idesc);
              }
            }
          } else {
            for (int gi = 0; gi < cnt; ++gi, a_lo += da_step, b_lo += db_step) {
              if (first) {
                tc_mma_i8_halves<0>(tmem_d, a_lo, a_hi, b_lo, b_hi, p.idesc);
                first = false;
              } else {
                tc_mma_i8_halves<1>(tmem_d, a_lo, a_hi, b_lo, b_hi, p.idesc);
              }
              for (int k = 1; k < ksteps; ++k) tc_mma_i8_halves<1>(tmem_d, a_lo + 2u * k, a_hi, b_lo + 2u * k, b_hi, p.idesc);
            }
          }
          tc_commit(smem_u32(&hdr->empty[s]));
        }
        __syncwarp();
        accumulate = 1;
        TC_TRACE(1, it, 1);
        if (++s == static_cast<uint32_t>(p.stages)) { s = 0; ph ^= 1; }
      }
      if (ok && elect_one()) {
        tc_commit(smem_u32(&hdr->tmem_full[a]));
        if (two) tc_commit(smem_u32(&hdr->tmem_full[a + 1]));
      }
      __syncwarp();
    }
  } else if (FUSE && warp == 3) {
    // ------------------------------------------------------------ residual producer (FUSE)
    // The residual tile of the Add (same rows and columns as the output tile) is brought into the
    // staging memory by TMA, two tiles deep, so that the epilogue reads it from shared memory.
    // First of all the Add's 64 KB table (a constant of the graph, so no waiting for earlier kernels): four bulk copies
    // that land while the first tiles are loaded and multiplied; the epilogue warps wait for them before their first
    // look-up.  (Copied by the epilogue threads themselves with ordinary loads, the table kept them from their first
    // tile for about five microseconds of every launch.)
    if (elect_one()) {
      const uint32_t full = smem_u32(&hdr->tab_full);
      mbar_arrive_expect_tx(full, 65536u);
      for (int q = 0; q < 4; ++q) bulk_load(smem_u32(add_tab) + q * 16384u, p.ep.add_table + q * 16384, 16384u, full);
    }
    __syncwarp();
    if (p.res_span) {
      pdl_wait();   // the residual is an earlier kernel's output
      const int span = p.res_span;
      int nload = 0;
      for (int blk = 0; blk * span < p.BNd; ++blk)
        if (n_tile * p.BNd + blk * span < p.Ocp) ++nload;
      const uint32_t box_bytes = static_cast<uint32_t>(p.conv ? p.TW * p.TH * p.TN : kBlockM) * span;
      bool ok = true;
      int m_tile = m_tile0, j = 0;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, m_tile += m_step, ++j) {
        const uint32_t b = j & 1, ph = (j >> 1) & 1;
        ok = mbar_wait(smem_u32(&hdr->res_empty[b]), ph ^ 1, abort_flag, p.status, 6, p.wait_limit);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (elect_one()) {
          const uint32_t full = smem_u32(&hdr->res_full[b]);
          mbar_arrive_expect_tx(full, static_cast<uint32_t>(nload) * box_bytes);
          uint32_t dst = smem_u32(staging + b * staging_bytes);
          for (int blk = 0; blk < nload; ++blk, dst += static_cast<uint32_t>(kBlockM) * span) {
            const int col = n_tile * p.BNd + blk * span;
            if (p.conv) {
              const int rest = m_tile / p.tiles_w;
              tma_load_4d(dst, &map_d, col, (m_tile % p.tiles_w) * p.TW, (rest % p.tiles_h) * p.TH, (rest / p.tiles_h) * p.TN, full);
            } else {
              tma_load_2d(dst, &map_d, col, m_tile * kBlockM, full);
            }
          }
        }
        __syncwarp();
      }
    }
  } else if (warp >= kFirstEpilogueWarp) {
    // ------------------------------------------------------------ epilogue
    // The epilogue's constants (this N tile's folded bias and scales) are staged by the epilogue warps themselves,
    // behind a barrier of their own: the producers and the MMA warp are already at work on the first tile meanwhile.
    for (int i = threadIdx.x - kFirstEpilogueWarp * 32; i < p.BNd; i += kEpilogueThreads) {
      const int oc = n_tile * p.BNd + i;
      hdr->bias[i] = oc < p.Ocp ? p.ep.bias_full[oc] : 0;
      hdr->scale[i] = oc < p.Ocp ? p.ep.acc_scale[oc] : 0.0f;
    }
    epilogue_barrier();
    const int ew = warp - kFirstEpilogueWarp;     // 0..15
    const int quarter = warp & 3;                 // TMEM lanes [32*quarter, +32) belong to this warp
    const int col_group = ew >> 2;                // this warp takes 16-column chunks col_group, col_group+4, ...
    const int row_in_tile = quarter * 32 + lane;
    const bool store_issuer = threadIdx.x == kFirstEpilogueWarp * 32;
    const OutQuant oq = p.ep.out;
    const RequantConsts rc = make_requant_consts(oq, p.exact_only);
    // position of this thread's 16-byte chunks inside a staging column block
    const int span_b = p.store_span;
    const int span_r = FUSE ? p.res_span : 0;        // never both: a fused Add stores directly
    const int span_s = span_b ? span_b : span_r;     // layout of the staging memory either way
    const int span_shift = span_s == 128 ? 7 : (span_s == 64 ? 6 : 5);
    const int swz = span_s == 128 ? (row_in_tile & 7) : span_s == 64 ? ((row_in_tile >> 1) & 3) : ((row_in_tile >> 2) & 1);
    int j = 0;
    // Once a wait has given up (alive == false) a thread does no more work, but it keeps running the
    // loop and both barriers of every tile, so the other epilogue threads never wait for it.
    // Output row of this thread in M tile m_tile (-1 outside the tensor) and, for a border pixel of a padded
    // convolution, the row of corrections of its class.
    auto locate = [&](int m_tile, long long& row, const int32_t*& corr_row) {
      row = -1;
      corr_row = nullptr;
      if (p.conv) {
        if (!span_b || FUSE || (EXTRA && p.ep.border_corr)) {
          const int tw = m_tile % p.tiles_w, rest = m_tile / p.tiles_w;
          const int th = rest % p.tiles_h, tn = rest / p.tiles_h;
          const int i = row_in_tile % p.TW, r2 = row_in_tile / p.TW;
          const int jh = r2 % p.TH, l = r2 / p.TH;
          const int wo = tw * p.TW + i, ho = th * p.TH + jh, n = tn * p.TN + l;
          if (l < p.TN && wo < p.Wo && ho < p.Ho && n < p.Nimg) {
            row = (static_cast<long long>(n) * p.Ho + ho) * p.Wo + wo;
            if (EXTRA && p.ep.border_corr) {
              const int cls = __ldg(p.ep.row_class + ho) * p.ep.n_col_classes + __ldg(p.ep.col_class + wo);
              if (cls) corr_row = p.ep.border_corr + static_cast<size_t>(cls) * p.Ocp + n_tile * p.BNd;
            }
          }
        }
      } else if (!span_b || FUSE) {
        row = static_cast<long long>(m_tile) * kBlockM + row_in_tile;
        if (row >= p.M) row = -1;
      }
    };
    bool alive = true;
    bool table_ready = !FUSE;
    const int j_step = p.teams ? kGroups : 1;               // team mode: warp group col_group takes tiles j = col_group (mod kGroups)
    const int c_first = p.teams ? 0 : col_group * 16;       // and all of their chunks
    const int c_step = p.teams ? 16 : kGroups * 16;
    j = p.teams ? col_group : 0;
    for (int tile = blockIdx.x + j * static_cast<int>(gridDim.x); tile < num_tiles; tile += j_step * static_cast<int>(gridDim.x), j += j_step) {
      const int m_tile = m_tile0 + j * m_step;
      const uint32_t a = j & ((1 << p.acc_shift) - 1), aph = (j >> p.acc_shift) & 1;
      uint8_t* stage_out = staging + (j & 1) * staging_bytes;
      long long row;                 // direct-store path: output row (pixel index into D), -1 outside the tensor
      const int32_t* corr_row;       // border pixels of a padded convolution: their correction, this N tile
      locate(m_tile, row, corr_row);
      TC_EPI(j, 0);
      if (alive) alive = mbar_wait(smem_u32(&hdr->tmem_full[a]), aph, abort_flag, p.status, 4, p.wait_limit);
      alive = __all_sync(0xffffffffu, alive);   // the TMEM loads below are warp-wide
      if (!alive) {
        if (span_b) epilogue_barrier();
        continue;
      }
      TC_EPI(j, 1);
      if (span_r) {
        alive = mbar_wait(smem_u32(&hdr->res_full[j & 1]), (j >> 1) & 1, abort_flag, p.status, 7, p.wait_limit);
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) continue;
      }
      if (!table_ready) {   // first tile of a fused Add: the table's bulk copies
        alive = mbar_wait(smem_u32(&hdr->tab_full), 0, abort_flag, p.status, 10, p.wait_limit);
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) continue;
        table_ready = true;
      }
      TC_EPI(j, 2);
      if (warp == kFirstEpilogueWarp && lane == 0) TC_TRACE(2, j, 0);
      tc_fence_after();
      const uint32_t taddr = tmem_base + a * p.acc_stride + (static_cast<uint32_t>(quarter * 32) << 16);
      // Chunks col_group, col_group + 4, ... of 16 columns; the TMEM load of the next chunk is in flight
      // while the current one is requantized.
      int sub = 0;
      if (EXTRA && p.dz != 0) {
        // S = sum of this row's inputs: the accumulator column of the all-ones weight row
        int s_val;
        tc_ld_32x1(taddr + p.BNd, s_val);
        tc_ld_wait1(s_val);
        sub = p.dz * s_val;
      }
      auto emit = [&](const int (&acc)[16], int c0) {
        const int cbase = n_tile * p.BNd + c0;
        if (!span_b && (row < 0 || cbase + 16 > p.Ocp)) return;
        uint4 res16 = make_uint4(0, 0, 0, 0);
        if (FUSE) {
          if (span_r) {
            const int blk = c0 >> span_shift, chunk = (c0 & (span_r - 1)) >> 4;
            res16 = *reinterpret_cast<const uint4*>(staging + (j & 1) * staging_bytes + static_cast<size_t>(blk) * kBlockM * span_r +
                                                    row_in_tile * span_r + ((chunk ^ swz) << 4));
          } else if (row >= 0 && cbase + 16 <= p.Ocp) {
            res16 = __ldg(reinterpret_cast<const uint4*>(p.ep.add_residual + row * p.ldd + cbase));
          }
        }
#ifdef B2VX_ABL_NOREQ
        uint4 out16 = make_uint4(acc[0] ^ acc[4] ^ acc[8] ^ acc[12], acc[1] ^ acc[5] ^ acc[9] ^ acc[13], acc[2] ^ acc[6] ^ acc[10] ^ acc[14],
                                 acc[3] ^ acc[7] ^ acc[11] ^ acc[15]);
#else
        uint4 out16 = requant_chunk16<EXTRA>(acc, &hdr->bias[c0], &hdr->scale[c0], rc, sub,
                                             (corr_row && cbase + 16 <= p.Ocp) ? corr_row + c0 : nullptr);
#endif
#ifdef B2VX_ABL_NOLUT
        if (FUSE) { out16.x ^= res16.x; out16.y ^= res16.y; out16.z ^= res16.z; out16.w ^= res16.w; }
        else
#endif
        if (FUSE) {
          out16.x = add_lut_word(out16.x, res16.x, add_tab);
          out16.y = add_lut_word(out16.y, res16.y, add_tab);
          out16.z = add_lut_word(out16.z, res16.z, add_tab);
          out16.w = add_lut_word(out16.w, res16.w, add_tab);
        }
        if (span_b) {
          const int blk = c0 >> span_shift, chunk = (c0 & (span_b - 1)) >> 4;   // span_b is 32, 64 or 128
          *reinterpret_cast<uint4*>(stage_out + static_cast<size_t>(blk) * kBlockM * span_b + row_in_tile * span_b +
                                    ((chunk ^ swz) << 4)) = out16;
        } else {
          *reinterpret_cast<uint4*>(p.D + row * p.ldd + cbase) = out16;
        }
      };
      {
        int acc_a[16], acc_b[16];
        int c0 = c_first;
        if (c0 < p.BNd) tc_ld_32x16(taddr + c0, acc_a);
        while (c0 < p.BNd) {
          tc_ld_wait(acc_a);
          if (c0 + c_step < p.BNd) tc_ld_32x16(taddr + c0 + c_step, acc_b);
          emit(acc_a, c0);
          c0 += c_step;
          if (c0 >= p.BNd) break;
          tc_ld_wait(acc_b);
          if (c0 + c_step < p.BNd) tc_ld_32x16(taddr + c0 + c_step, acc_a);
          emit(acc_b, c0);
          c0 += c_step;
        }
      }
      TC_EPI(j, 3);
      // accumulator buffer (and residual buffer) free again
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&hdr->tmem_empty[a]));
        if (span_r) mbar_arrive(smem_u32(&hdr->res_empty[j & 1]));
      }
      if (span_b) {
        // One barrier per tile.  Before it, the issuer makes sure the previous tile's store has read
        // its staging buffer (it was issued a whole tile ago): after the barrier every thread may
        // write that buffer for the next tile, and the issuer stores the tile just written.
        fence_smem_to_async();
        if (store_issuer) tma_store_wait_read<0>();
        epilogue_barrier();
        if (store_issuer) {
          const int nblk = p.BNd / span_b;
          for (int blk = 0; blk < nblk; ++blk) {
            const int col = n_tile * p.BNd + blk * span_b;
            if (col >= p.Ocp) break;
            const uint32_t src = smem_u32(stage_out + static_cast<size_t>(blk) * kBlockM * span_b);
            if (p.conv) {
              const int rest = m_tile / p.tiles_w;
              tma_store_4d(&map_d, src, col, (m_tile % p.tiles_w) * p.TW, (rest % p.tiles_h) * p.TH, (rest / p.tiles_h) * p.TN);
            }
            else tma_store_2d(&map_d, src, col, m_tile * kBlockM);
          }
          tma_store_commit();
        }
      }
      if (warp == kFirstEpilogueWarp && lane == 0) TC_TRACE(2, j, 1);
    }
    // The staging buffers only have to stay intact until the last store has read them; the writes
    // themselves are complete, like any other store, when the grid is.
    if (store_issuer) tma_store_wait_read<0>();
  }

  // ---------------------------------------------------------------- common exit
  tc_fence_before();
  __syncthreads();
  TC_MARK(2);
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(p.tmem_cols))
                 : "memory");
  }
}

// ---- issue-rate microbenchmark of the int8 tensor pipe ----------------------------------------
// One CTA per SM; operands (pseudo-random bytes) stay in shared memory, one thread issues `iters` rounds of
// four M=128, N=256, K=32 tcgen05.mma.kind::i8 (one 128-byte K block) into two alternating accumulators and
// commits every round to an mbarrier it waits on two rounds later, so the pipe always has work queued.  No
// loads from global memory and no epilogue: what is timed is the rate at which the tensor pipe retires MMAs.
// n, span: the instruction's N and the operands' swizzle span in bytes (256 and 128 for the peak; other values show what
// narrower instructions and narrower spans deliver: B2VX_PEAK_N / B2VX_PEAK_SPAN at the host entry).
__global__ void __launch_bounds__(128, 1) int8_peak_kernel(int iters, int n, int span, int* status) {
  extern __shared__ uint8_t peak_smem[];
  __shared__ unsigned long long bars[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const uint32_t base = (smem_u32(peak_smem) + 1023u) & ~1023u;
  uint8_t* tiles = peak_smem + (base - smem_u32(peak_smem));
  uint32_t h = 0x9E3779B9u * (threadIdx.x + 1u) + blockIdx.x;
  for (uint32_t i = threadIdx.x; i < (128u + 256u) * 128u / 4u; i += blockDim.x) {
    h = h * 1664525u + 1013904223u;
    reinterpret_cast<uint32_t*>(tiles)[i] = h;
  }
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars[0]), 1);
    mbar_init(smem_u32(&bars[1]), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the operand bytes were written with ordinary stores
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = (2u << 4) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
    const uint32_t layout = span == 128 ? 2u : (span == 64 ? 4u : 6u);
    const uint64_t da = make_smem_desc(base, 8u * span, layout), db = make_smem_desc(base + 128u * 128u, 8u * span, layout);
    const int ksteps = span >> 5;
    bool ok = true;
    for (int it = 0; it < iters && ok; ++it) {
      const int b = it & 1;
      if (it >= 2) ok = mbar_wait(smem_u32(&bars[b]), ((it - 2) >> 1) & 1, &abort_flag, status, 9);
      if (!ok) break;
      tc_fence_after();
      for (int k = 0; k < 4; ++k) {
        const int kk = k & (ksteps - 1);   // four instructions per round whatever the span (ksteps is 1, 2 or 4)
        tc_mma_i8(tmem + b * 256, da + static_cast<uint64_t>(kk * 2), db + static_cast<uint64_t>(kk * 2), idesc, 1);
      }
      tc_commit(smem_u32(&bars[b]));
    }
    for (int it = max(0, iters - 2); it < iters && ok; ++it) ok = mbar_wait(smem_u32(&bars[it & 1]), (it >> 1) & 1, &abort_flag, status, 9);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

CUtensorMapSwizzle swizzle_of(int span) {
  return span == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (span == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

// uint8 tensor of rank 2 or 4, dense (stride of dim i+1 = stride of dim i * dims[i])
bool encode_u8(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint32_t* box, const uint32_t* estr,
               CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t d[4], strides[3];
  cuuint32_t b[4], e[4];
  uint64_t pitch = 1;
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = estr ? estr[i] : 1;
    pitch *= dims[i];
    if (i + 1 < rank) strides[i] = pitch;
  }
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, strides, b, e,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

struct GemmTcPlan {
  CUtensorMap map_a;
  CUtensorMap map_b;
  CUtensorMap map_d;
  GemmParams params;
  int grid;
  size_t smem;
};

int gemm_tc_available(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return 0;
  return prop.major == 10 && get_encode_fn() != nullptr;
}

namespace {

// Everything of a plan that does not depend on how A is addressed: N tiling, K block / swizzle mode,
// output staging, stage count, TMEM columns, instruction descriptor, the B tensor map.
// Kspan is the K extent one tap (or the whole GEMM) covers, used to pick BK.
// halo_w, halo_h: extent in pixels of the input patch (tile + halo) the caller would load per channel block if the plan
// turns out to allow the halo mode of the implicit convolution (0: not asked for).
bool finish_plan(GemmTcPlan* plan, const int8_t* B, int a_signed, int Np, int Kp, int Kspan, int taps, int ldd,
                 const ContractEpilogue& e, void* D, int* status, const char** why, const GemmTcTiling* tiling, int halo_w = 0,
                 int halo_h = 0, bool want_pair = false, bool wide_teams = false) {
  GemmParams& p = plan->params;
  p.Ocp = ldd;
  p.ldd = ldd;
  if (tiling) {
    p.n_tiles = tiling->n_tiles;
    p.BN = tiling->rows;
    p.BNd = tiling->data;
    if (p.BN > 256 || (p.BN & 15) || (p.BNd & 15) || p.BNd < 16 || p.BNd > p.BN) { *why = "gemm_tc: bad N tiling"; return false; }
  } else {
    p.n_tiles = (Np + 255) / 256;
    p.BN = (((Np + p.n_tiles - 1) / p.n_tiles) + 15) & ~15;
    p.BNd = p.BN;
  }
  if (p.n_tiles * p.BN != Np) { *why = "gemm_tc: weight rows must be packed to n_tiles*BN"; return false; }
  p.dz = e.dz_uniform;
  if (p.dz != 0 && p.BNd == p.BN) { *why = "gemm_tc: a weight zero point needs the ones row in every N tile"; return false; }
  // K block: the swizzle span (32/64/128 bytes) that wastes the least tail.
  int best_bk = 32;
  long long best_cost = -1;
  for (int bk : {128, 64, 32}) {
    const long long cost = static_cast<long long>((Kspan + bk - 1) / bk) * bk;
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_bk = bk; }
  }
  p.BK = best_bk;
  p.layout_type = p.BK == 128 ? 2u : (p.BK == 64 ? 4u : 6u);
  p.sbo = 8u * p.BK;
  // Output staging for the TMA store: column blocks as wide as the widest swizzle span dividing BN.
  p.store_span = p.BNd % 128 == 0 ? 128 : (p.BNd % 64 == 0 ? 64 : (p.BNd % 32 == 0 ? 32 : 0));
  // Measured over the ResNet-50 layer shapes, threads storing their 16-byte pieces themselves beat the
  // staged TMA store (no CTA-wide barrier per tile, epilogue warps drift apart and overlap tiles, and
  // the staging memory goes to the operand ring instead), so that is the default;
  // B2VX_TC_STORE=tma selects the staged store.
  static const bool tma_store = [] { const char* e = std::getenv("B2VX_TC_STORE"); return e && std::strcmp(e, "tma") == 0; }();
  p.res_span = e.add_residual != nullptr ? p.store_span : 0;
  if (!tma_store || e.add_residual != nullptr) p.store_span = 0;
  const size_t add_table_bytes = e.add_residual != nullptr ? 65536 : 0;
  static const bool no_teams = [] { const char* e2 = std::getenv("B2VX_TC_TEAMS"); return e2 && std::strcmp(e2, "0") == 0; }();
  // (wide_teams: the caller found the launch bound by its epilogue, short K and many tiles per CTA, so tiles of up to 128
  // columns also go one per warp group: four tiles in flight instead of four passes over every tile)
  p.teams = ((p.BNd <= 64 || (wide_teams && p.BN <= 128)) && p.store_span == 0 && !no_teams) ? kGroups : 0;
  if (p.teams) p.res_span = 0;   // four tiles in flight do not fit the two residual buffers: threads load their pieces
  if (p.res_span) {
    // The Add's table and two residual tiles leave less for the operand ring: three stages must remain,
    // with 64-byte K blocks if 128-byte ones do not fit (these layers are bound by their epilogue, not by
    // the main loop); failing that the epilogue threads load their residual pieces themselves.
    const size_t left = kSmemBudget - 2048 - sizeof(SmemHeader) - add_table_bytes - 2 * static_cast<size_t>(kBlockM) * p.BNd;
    if (left < 3 * static_cast<size_t>(kBlockM + p.BN) * p.BK && p.BK == 128) {
      p.BK = 64;
      p.layout_type = 4u;
      p.sbo = 8u * p.BK;
    }
    if (left < 3 * static_cast<size_t>(kBlockM + p.BN) * p.BK) p.res_span = 0;
  }
  const int kblocks_per_tile = taps * ((Kspan + p.BK - 1) / p.BK);
  const size_t staging = (p.store_span || p.res_span) ? 2 * static_cast<size_t>(kBlockM) * p.BNd : 0;
  // A and B tiles are whole swizzle atoms (8 rows x BK bytes; BN and 128 are multiples of 8), so every
  // tile start keeps the alignment its swizzle pattern repeats on (8*BK bytes) relative to the 1024-byte
  // aligned start of the ring.  Several k-blocks share a stage (one barrier round trip) when they are
  // small: up to 64 KiB per stage.
  // Resident weights: the whole [BN x K] tile of this CTA's N tile when it is small (B2VX_TC_BRES=0 disables).
  static const bool no_bres = [] { const char* e2 = std::getenv("B2VX_TC_BRES"); return e2 && std::strcmp(e2, "0") == 0; }();
  const size_t b_all = static_cast<size_t>(kblocks_per_tile) * p.BN * p.BK;
  // (beside a fused Add's table and residual tiles only up to 32 KB)
  p.b_resident = (!no_bres && b_all <= (e.add_residual != nullptr ? 32u : 72u) * 1024) ? 1 : 0;
  const size_t bres = p.b_resident ? ((b_all + 1023) & ~static_cast<size_t>(1023)) : 0;
  // Halo mode: weights resident, 64-byte K blocks (the swizzle mode whose shifted views were verified on the device);
  // B2VX_TC_HALO=0 keeps one shifted TMA box per tap.
  static const bool no_halo = [] { const char* e2 = std::getenv("B2VX_TC_HALO"); return e2 && std::strcmp(e2, "0") == 0; }();
  p.halo = (halo_w > 0 && !no_halo && p.b_resident && p.BK == 64 && e.add_residual == nullptr) ? 1 : 0;
  p.halo_w = p.halo ? halo_w : 0;
  p.a_stage_bytes = p.halo ? static_cast<uint32_t>((static_cast<size_t>(halo_w) * halo_h * p.BK + 1023) & ~static_cast<size_t>(1023)) : 0u;
  p.num_kb_b = kblocks_per_tile;
  // Pair mode (see GemmParams): asked for by the caller where the K loop is long and every CTA has several tiles; needs
  // the weights in the ring, exactly two accumulator buffers (tiles wider than 128 columns) and no fused Add.
  // B2VX_TC_PAIR=0 disables.
  const char* pair_env = std::getenv("B2VX_TC_PAIR");   // read per plan, so that one process can build both forms
  const bool no_pair = pair_env && std::strcmp(pair_env, "0") == 0;
  p.pair = (want_pair && !no_pair && !p.halo && !p.b_resident && !p.teams && e.add_residual == nullptr && p.BN > 128) ? 1 : 0;
  const size_t sub_bytes = p.halo ? p.a_stage_bytes : static_cast<size_t>((p.pair ? 2 : 1) * kBlockM + (p.b_resident ? 0 : p.BN)) * p.BK;
  const size_t ring_budget = kSmemBudget - 2048 - sizeof(SmemHeader) - staging - add_table_bytes - bres;
  int group = static_cast<int>((64 * 1024) / sub_bytes);
  if (p.halo) group = 1;
  if (group > kblocks_per_tile) group = kblocks_per_tile;
  if (group > kMaxGroup) group = kMaxGroup;
  if (group < 1) group = 1;
  while (group > 1 && ring_budget / (sub_bytes * group) < 3) --group;
  p.group = group;
  const size_t stage_bytes = sub_bytes * group;
  int stages = static_cast<int>(ring_budget / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) { *why = "gemm_tc: tile does not fit shared memory"; return false; }
  p.stages = stages;
  // the epilogue reads 16 columns at a time; buffers start on 32-column boundaries
  // As many accumulator buffers as the 512 TMEM columns hold (2, 4 or 8): with narrow tiles the
  // epilogue of a tile is a latency chain, and more tiles in flight hide it.
  p.acc_stride = (p.BN + 31) & ~31;
  p.acc_shift = 1;
  while (p.acc_shift < 3 && (2 << p.acc_shift) * p.acc_stride <= 512) ++p.acc_shift;
  if (p.teams && (1 << p.acc_shift) < kGroups) p.teams = 0;   // every team's tile needs an accumulator buffer
  int cols = 32;
  while (cols < (1 << p.acc_shift) * p.acc_stride) cols <<= 1;
  p.tmem_cols = cols;
  p.idesc = (2u << 4) | (static_cast<uint32_t>(a_signed ? 1 : 0) << 7) | (1u << 10) |
            (static_cast<uint32_t>(p.BN >> 3) << 17) | (static_cast<uint32_t>(kBlockM >> 4) << 24);
  p.ep = e;
  p.exact_only = e.exact_only;
  p.wait_limit = kWaitLimitCycles;
  p.tx_extra = 0;
  p.D = static_cast<uint8_t*>(D);
  p.status = status;
  const uint64_t bdims[2] = {static_cast<uint64_t>(Kp), static_cast<uint64_t>(Np)};
  const uint32_t bbox[2] = {static_cast<uint32_t>(p.BK), static_cast<uint32_t>(p.BN)};
  if (!encode_u8(&plan->map_b, B, 2, bdims, bbox, nullptr, swizzle_of(p.BK))) {
    *why = "gemm_tc: cuTensorMapEncodeTiled failed for the weights";
    return false;
  }
  size_t smem = ((static_cast<size_t>(stages) * stage_bytes + 1023) & ~static_cast<size_t>(1023)) + bres + staging + add_table_bytes + sizeof(SmemHeader) + 1024;
  if (smem < static_cast<size_t>(kMinDynSmem)) smem = kMinDynSmem;
  plan->smem = smem;
  // the attribute belongs to the function on one device: set it once per device of this process
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_i8_tc_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_i8_tc_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_i8_tc_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_i8_tc_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      *why = "gemm_tc: cannot raise the dynamic shared memory limit";
      return false;
    }
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  return true;
}

void set_grid(GemmTcPlan* plan) {
  GemmParams& p = plan->params;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // a multiple of n_tiles, so that every CTA works on one N tile only
  const int tiles = p.m_tiles * p.n_tiles;
  int grid = (sms / p.n_tiles) * p.n_tiles;
  if (grid < p.n_tiles) grid = p.n_tiles;
  if (grid > tiles) grid = tiles;
  plan->grid = grid;
}

}  // namespace

GemmTcPlan* gemm_tc_plan_create(const void* A, int a_signed, const int8_t* B, int M, int Np, int Kp, int Oc, void* D,
                                int ldd, int d_signed, const ContractEpilogue& e, int* status, char* err,
                                size_t err_len, const GemmTcTiling* tiling) {
  (void)Oc;
  (void)d_signed;
  auto fail = [&](const char* msg) -> GemmTcPlan* {
    if (err && err_len) std::snprintf(err, err_len, "%s", msg);
    return nullptr;
  };
  if (M <= 0 || Np <= 0 || Kp <= 0 || (Kp & 15) || (ldd & 15) || (Np & 15)) return fail("gemm_tc: sizes must be positive multiples of 16");
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(D) & 15))
    return fail("gemm_tc: operands must be 16-byte aligned");
  if (e.dz != nullptr || e.tapc != nullptr || e.out_is_float) return fail("gemm_tc: epilogue form not supported");

  GemmTcPlan* plan = new GemmTcPlan();
  GemmParams& p = plan->params;
  std::memset(&p, 0, sizeof(p));
  std::memset(&plan->map_d, 0, sizeof(plan->map_d));
  const char* why = "";
  // pair mode where the main loop dwarfs the epilogue (K of 4096 or more) and there are at least two tiles per SM
  int sms = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long tiles_256 = static_cast<long long>((M + kBlockM - 1) / kBlockM) * ((Np + 255) / 256);
  const bool want_pair = Kp >= 4096 && tiles_256 >= 2LL * sms;
  const bool wide_teams = Kp <= 128 && static_cast<long long>((M + kBlockM - 1) / kBlockM) >= 8LL * sms;
  if (!finish_plan(plan, B, a_signed, Np, Kp, Kp, 1, ldd, e, D, status, &why, tiling, 0, 0, want_pair, wide_teams)) {
    delete plan;
    return fail(why);
  }
  p.M = M;
  p.num_kb = (Kp + p.BK - 1) / p.BK;
  p.m_tiles = (M + kBlockM - 1) / kBlockM;
  p.a_tx_bytes = static_cast<uint32_t>(kBlockM) * p.BK;
  const uint64_t adims[2] = {static_cast<uint64_t>(Kp), static_cast<uint64_t>(M)};
  const uint32_t abox[2] = {static_cast<uint32_t>(p.BK), kBlockM};
  bool ok = encode_u8(&plan->map_a, A, 2, adims, abox, nullptr, swizzle_of(p.BK));
  if (ok && (p.store_span || p.res_span)) {
    // the output tile for the staged store, or (fused Add) the residual tile of the same geometry
    const int span = p.store_span ? p.store_span : p.res_span;
    const uint64_t ddims[2] = {static_cast<uint64_t>(ldd), static_cast<uint64_t>(M)};
    const uint32_t dbox[2] = {static_cast<uint32_t>(span), kBlockM};
    ok = encode_u8(&plan->map_d, p.store_span ? D : static_cast<const void*>(e.add_residual), 2, ddims, dbox, nullptr, swizzle_of(span));
  }
  if (!ok) {
    delete plan;
    return fail("gemm_tc: cuTensorMapEncodeTiled failed");
  }
  set_grid(plan);
  return plan;
}

GemmTcPlan* gemm_tc_conv_plan_create(const void* X, int x_signed, const int8_t* B, const ConvGeom& g, int Np, void* D,
                                     const ContractEpilogue& e, int* status, char* err, size_t err_len,
                                     const GemmTcTiling* tiling) {
  auto fail = [&](const char* msg) -> GemmTcPlan* {
    if (err && err_len) std::snprintf(err, err_len, "%s", msg);
    return nullptr;
  };
  if ((g.Cp & 15) || (g.Ocp & 15) || (Np & 15)) return fail("gemm_tc conv: channel counts must be padded to 16");
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(D) & 15))
    return fail("gemm_tc conv: operands must be 16-byte aligned");
  if (e.dz != nullptr || e.tapc != nullptr || e.out_is_float) return fail("gemm_tc conv: epilogue form not supported");

  GemmTcPlan* plan = new GemmTcPlan();
  GemmParams& p = plan->params;
  std::memset(&p, 0, sizeof(p));
  std::memset(&plan->map_d, 0, sizeof(plan->map_d));
  const char* why = "";
  const int Kp = g.kh * g.kw * g.Cp;
  // Halo mode (see GemmParams): a tile is 8 x 16 output pixels of one image.  Asked for when the convolution has more
  // than one tap, stride and dilation 1, and tiles of that shape waste at most 15 % of their rows on this output size.
  int halo_w = 0, halo_h = 0;
  if (g.kh * g.kw > 1 && g.sx == 1 && g.sy == 1 && g.dx == 1 && g.dy == 1 && g.kw <= 16 && g.kh <= 16) {
    const double covered = static_cast<double>((g.Wo + 7) / 8 * 8) * ((g.Ho + 15) / 16 * 16);
    if (static_cast<double>(g.Wo) * g.Ho >= 0.85 * covered) { halo_w = 8 + g.kw - 1; halo_h = 16 + g.kh - 1; }
  }
  if (!finish_plan(plan, B, x_signed, Np, Kp, g.Cp, g.kh * g.kw, g.Ocp, e, D, status, &why, tiling, halo_w, halo_h)) {
    delete plan;
    return fail(why);
  }
  // M tile = TW x TH x TN output pixels, at most 128: the shape that leaves the fewest tile rows unused.
  int bw = 1, bh = 1, bn = 1;
  double best = -1.0;
  for (int tw = 1; tw <= g.Wo && tw <= kBlockM; ++tw) {
    for (int th = 1; th <= g.Ho && tw * th <= kBlockM; ++th) {
      int tn = kBlockM / (tw * th);
      if (tn > g.N) tn = g.N;
      if (tn < 1) continue;
      // the box extent along a strided axis is (T-1)*stride+1 elements and may not exceed 256
      if ((tw - 1) * g.sx + 1 > 256 || (th - 1) * g.sy + 1 > 256) continue;
      const long long tiles = static_cast<long long>((g.Wo + tw - 1) / tw) * ((g.Ho + th - 1) / th) * ((g.N + tn - 1) / tn);
      const double eff = static_cast<double>(g.Wo) * g.Ho * g.N / (static_cast<double>(tiles) * kBlockM);
      // prefer wider rows at equal efficiency: longer contiguous runs per TMA box
      if (eff > best + 1e-9 || (eff > best - 1e-9 && tw > bw)) { best = eff; bw = tw; bh = th; bn = tn; }
    }
  }
  if (p.halo) { bw = 8; bh = 16; bn = 1; }
  p.conv = 1;
  p.TW = bw; p.TH = bh; p.TN = bn;
  p.tiles_w = (g.Wo + bw - 1) / bw;
  p.tiles_h = (g.Ho + bh - 1) / bh;
  const int tiles_n = (g.N + bn - 1) / bn;
  p.m_tiles = p.tiles_w * p.tiles_h * tiles_n;
  p.M = g.N * g.Ho * g.Wo;
  p.Wo = g.Wo; p.Ho = g.Ho; p.Nimg = g.N;
  p.kw = g.kw; p.sx = g.sx; p.sy = g.sy; p.dx = g.dx; p.dy = g.dy; p.pl = g.pl; p.pt = g.pt;
  p.Cp = g.Cp;
  p.cblocks = (g.Cp + p.BK - 1) / p.BK;
  p.halo_kh = g.kh;
  p.num_kb = p.halo ? p.cblocks : g.kh * g.kw * p.cblocks;   // stages per tile: one patch per channel block, or one box per tap and block
  p.a_tx_bytes = p.halo ? static_cast<uint32_t>(halo_w * halo_h) * p.BK : static_cast<uint32_t>(bw * bh * bn) * p.BK;
  const uint64_t dims[4] = {static_cast<uint64_t>(g.Cp), static_cast<uint64_t>(g.W), static_cast<uint64_t>(g.H), static_cast<uint64_t>(g.N)};
  const uint32_t box[4] = {static_cast<uint32_t>(p.BK), static_cast<uint32_t>(p.halo ? halo_w : (bw - 1) * g.sx + 1),
                           static_cast<uint32_t>(p.halo ? halo_h : (bh - 1) * g.sy + 1), static_cast<uint32_t>(bn)};
  const uint32_t estr[4] = {1, static_cast<uint32_t>(g.sx), static_cast<uint32_t>(g.sy), 1};
  bool ok = encode_u8(&plan->map_a, X, 4, dims, box, estr, swizzle_of(p.BK));
  if (ok && (p.store_span || p.res_span)) {
    const int span = p.store_span ? p.store_span : p.res_span;
    const uint64_t ddims[4] = {static_cast<uint64_t>(g.Ocp), static_cast<uint64_t>(g.Wo), static_cast<uint64_t>(g.Ho), static_cast<uint64_t>(g.N)};
    const uint32_t dbox[4] = {static_cast<uint32_t>(span), static_cast<uint32_t>(bw), static_cast<uint32_t>(bh), static_cast<uint32_t>(bn)};
    ok = encode_u8(&plan->map_d, p.store_span ? D : static_cast<const void*>(e.add_residual), 4, ddims, dbox, nullptr, swizzle_of(span));
  }
  if (!ok) {
    delete plan;
    return fail("gemm_tc conv: cuTensorMapEncodeTiled failed");
  }
  set_grid(plan);
  return plan;
}

GemmTcTiling gemm_tc_choose_tiling(long long M, int Ocp, int Kp, int with_s) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int extra = with_s ? 16 : 0;
  const int max_data = 256 - extra;
  const long long m_tiles = (M + kBlockM - 1) / kBlockM;
  const double rows = static_cast<double>(M < kBlockM ? M : kBlockM);
  GemmTcTiling best = {0, 0, 0};
  double best_time = 0.0;
  const bool l2_resident = (static_cast<double>(M) + Ocp) * Kp < 48.0e6;
  // B2VX_TC_BN=<width>: force the tile width (a tuning aid; ignored when it does not fit)
  static const int forced = [] { const char* e = std::getenv("B2VX_TC_BN"); return e ? std::atoi(e) : 0; }();
  if (forced >= 16 && forced <= max_data && (forced & 15) == 0) {
    const int nt = (Ocp + forced - 1) / forced;
    const int data = (((Ocp + nt - 1) / nt) + 15) & ~15;
    if (nt <= sms) {
      best.n_tiles = nt;
      best.data = data;
      best.rows = data + extra;
      return best;
    }
  }
  int last_data = 0;
  for (int nt = (Ocp + max_data - 1) / max_data; nt <= sms && nt * 16 <= Ocp + 15; ++nt) {
    const int data = (((Ocp + nt - 1) / nt) + 15) & ~15;
    if (data == last_data) continue;          // same tile width with more (empty) tiles
    last_data = data;
    if ((nt - 1) * data >= Ocp) continue;
    const int bn = data + extra;
    const long long tiles = m_tiles * nt;
    long long grid = (sms / nt) * nt;
    if (grid > tiles) grid = tiles;
    const double per_cta = static_cast<double>((tiles + grid - 1) / grid);
    // cycles per tile: tensor pipe (8192 MAC/clk), operand bytes (HBM share per SM when all SMs load,
    // more when few do), epilogue issue slots
    // (Measured with B2VX_PEAK_N: 4395 / 2572 / 1341 TOP/s at N = 256 / 128 / 64: an M = 128, K = 32 instruction takes
    // 134 / 115 / 110 cycles, i.e. at least about 110 whatever its N.  A model with that floor chose no better tilings on
    // the networks, whose narrow layers are bound elsewhere, so the term that was tuned on them stays.)
    const double mma = static_cast<double>(Kp) * bn / 64.0;
    // operands of a layer that fits the L2 several times over (a previous layer's output and a small
    // weight matrix) are served by the L2 at its per-SM rate; otherwise by the CTA's share of HBM
    double bytes_per_clk = 24.0 * sms / static_cast<double>(grid);
    if (bytes_per_clk > 64.0 || l2_resident) bytes_per_clk = 64.0;
    const double load = (rows + bn) * Kp / bytes_per_clk;
    // the epilogue takes the tile's 16-column chunks four at a time (one per column group), or, for tiles of at
    // most four chunks, a team of warps takes a whole tile: 9 cycles per column of a full group of four chunks
    const double chunks = data / 16.0;
    const double chunk_groups = data <= 64 ? chunks / 4.0 : std::ceil(chunks / 4.0);
    const double epi = 9.0 * 64.0 * chunk_groups + 300.0;
    const double mainloop = mma > load ? mma : load;
    const double steady = mainloop > epi ? mainloop : epi;
    const double time = mainloop + epi + (per_cta - 1.0) * steady;
    if (best.n_tiles == 0 || time < best_time * 0.97) {   // prefer wider tiles unless clearly slower
      best.n_tiles = nt;
      best.data = data;
      best.rows = bn;
      best_time = time;
    }
  }
  if (best.n_tiles == 0) {
    best.n_tiles = (Ocp + max_data - 1) / max_data;
    best.data = (((Ocp + best.n_tiles - 1) / best.n_tiles) + 15) & ~15;
    best.rows = best.data + extra;
  }
  return best;
}

// Dense int8 tensor-pipe rate of the current device in TOP/s (2 * MAC): best of `reps` launches of the
// microbenchmark above on every SM; *sm_count receives the number of SMs used.  Returns 0 on failure.
double gemm_tc_measure_int8_peak(int reps, int* sm_count, int* status) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0.0;
  const size_t smem = (128 + 256) * 128 + 1024;
  if (cudaFuncSetAttribute(int8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kMinDynSmem)) != cudaSuccess) return 0.0;
  (void)smem;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return 0.0;
  const int iters = 20000;   // x 4 MMAs of 128 x 256 x 32: about 10 ms per launch
  // diagnostic: another instruction width (a multiple of 16 up to 256) or operand swizzle span (32, 64, 128 bytes)
  int n = 256, span = 128;
  if (const char* v = std::getenv("B2VX_PEAK_N")) { const int t = std::atoi(v); if (t >= 16 && t <= 256 && t % 16 == 0) n = t; }
  if (const char* v = std::getenv("B2VX_PEAK_SPAN")) { const int t = std::atoi(v); if (t == 32 || t == 64 || t == 128) span = t; }
  double best = 0.0;
  for (int r = 0; r < reps + 1; ++r) {
    cudaEventRecord(e0, 0);
    int8_peak_kernel<<<sms, 128, kMinDynSmem, 0>>>(iters, n, span, status);   // kMinDynSmem keeps it to one CTA per SM
    cudaEventRecord(e1, 0);
    if (cudaEventSynchronize(e1) != cudaSuccess) { best = 0.0; break; }
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    const double tops = 2.0 * 128.0 * n * 128.0 * iters * sms / (ms * 1e-3) / 1e12;
    if (r > 0 && tops > best) best = tops;   // the first launch warms up
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (sm_count) *sm_count = sms;
  return cudaGetLastError() == cudaSuccess ? best : 0.0;
}

size_t gemm_tc_plan_bytes(void) { return sizeof(GemmTcPlan); }

// Same plan as gemm_tc_plan_create, but built inside caller-provided storage (no heap allocation);
// the caller must not pass it to gemm_tc_plan_destroy.
GemmTcPlan* gemm_tc_plan_build_in(void* storage, size_t storage_bytes, const void* A, int a_signed, const int8_t* B, int M,
                                  int Np, int Kp, void* D, int ldd, const ContractEpilogue& e, int* status, char* err,
                                  size_t err_len) {
  auto fail = [&](const char* msg) -> GemmTcPlan* {
    if (err && err_len) std::snprintf(err, err_len, "%s", msg);
    return nullptr;
  };
  if (!storage || storage_bytes < sizeof(GemmTcPlan) || (reinterpret_cast<uintptr_t>(storage) & 63))
    return fail("gemm_tc: plan storage too small or not 64-byte aligned");
  if (M <= 0 || Np <= 0 || Kp <= 0 || (Kp & 15) || (ldd & 15) || (Np & 15)) return fail("gemm_tc: sizes must be positive multiples of 16");
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(D) & 15))
    return fail("gemm_tc: operands must be 16-byte aligned");
  if (e.dz != nullptr || e.tapc != nullptr || e.out_is_float) return fail("gemm_tc: epilogue form not supported");
  GemmTcPlan* plan = static_cast<GemmTcPlan*>(storage);
  std::memset(plan, 0, sizeof(GemmTcPlan));
  GemmParams& p = plan->params;
  const char* why = "";
  if (!finish_plan(plan, B, a_signed, Np, Kp, Kp, 1, ldd, e, D, status, &why, nullptr)) return fail(why);
  p.M = M;
  p.num_kb = (Kp + p.BK - 1) / p.BK;
  p.m_tiles = (M + kBlockM - 1) / kBlockM;
  p.a_tx_bytes = static_cast<uint32_t>(kBlockM) * p.BK;
  const uint64_t adims[2] = {static_cast<uint64_t>(Kp), static_cast<uint64_t>(M)};
  const uint32_t abox[2] = {static_cast<uint32_t>(p.BK), kBlockM};
  bool ok = encode_u8(&plan->map_a, A, 2, adims, abox, nullptr, swizzle_of(p.BK));
  if (ok && (p.store_span || p.res_span)) {
    // the output tile for the staged store, or (fused Add) the residual tile of the same geometry
    const int span = p.store_span ? p.store_span : p.res_span;
    const uint64_t ddims[2] = {static_cast<uint64_t>(ldd), static_cast<uint64_t>(M)};
    const uint32_t dbox[2] = {static_cast<uint32_t>(span), kBlockM};
    ok = encode_u8(&plan->map_d, p.store_span ? D : static_cast<const void*>(e.add_residual), 2, ddims, dbox, nullptr, swizzle_of(span));
  }
  if (!ok) return fail("gemm_tc: cuTensorMapEncodeTiled failed");
  set_grid(plan);
  return plan;
}

void gemm_tc_plan_destroy(GemmTcPlan* p) { delete p; }

int gemm_tc_plan_is_halo(const GemmTcPlan* p) { return p && p->params.halo ? 1 : 0; }

cudaError_t gemm_tc_launch(const GemmTcPlan* plan, cudaStream_t s) {
#ifdef B2VX_TC_TRACE
  GemmTcPlan* mp = const_cast<GemmTcPlan*>(plan);
  if (!mp->params.trace) {
    cudaMalloc(reinterpret_cast<void**>(&mp->params.trace), (3 * 64 * 2 + 16 + 128) * sizeof(long long));
    cudaMemset(mp->params.trace, 0, (3 * 64 * 2 + 16 + 128) * sizeof(long long));
  }
#endif
  // Test aid: B2VX_TEST_STALL=<n> makes the first n launches of the process announce 16 bytes more than their loads
  // deliver and give up after about a millisecond, so that the path "a barrier wait ran out -> status word ->
  // B2VX_DEVICE_TIMEOUT" can be exercised without harming the GPU: every real load lands, the kernel leaves
  // through its common exit.  (Use with B2VX_CUDA_GRAPH=0: a captured launch would keep the stall.)
  static std::atomic<int> stall_left([] { const char* v = std::getenv("B2VX_TEST_STALL"); return v ? std::atoi(v) : 0; }());
  GemmTcPlan stalled;
  if (stall_left.load(std::memory_order_relaxed) > 0 && stall_left.fetch_sub(1) > 0) {
    stalled = *plan;
    stalled.params.wait_limit = 2000000LL;
    stalled.params.tx_extra = 16;
    plan = &stalled;
  }
  cudaError_t launched;
  const bool extra = plan->params.dz != 0 || plan->params.ep.border_corr != nullptr;
  const bool fuse = plan->params.ep.add_residual != nullptr;
#define B2VX_GEMM_LAUNCH(E_, F_) launch_pdl(gemm_i8_tc_kernel<E_, F_>, dim3(plan->grid), dim3(kThreadsTc), plan->smem, s, plan->map_a, \
                                            plan->map_b, plan->map_d, plan->params)
  if (fuse) launched = extra ? B2VX_GEMM_LAUNCH(true, true) : B2VX_GEMM_LAUNCH(false, true);
  else launched = extra ? B2VX_GEMM_LAUNCH(true, false) : B2VX_GEMM_LAUNCH(false, false);
#undef B2VX_GEMM_LAUNCH
  if (launched != cudaSuccess) return launched;
#ifdef B2VX_TC_TRACE
  {
    static int launches = 0;
    if (++launches == 3) {
      cudaStreamSynchronize(s);
      long long h[3 * 64 * 2 + 16 + 128];
      cudaMemcpy(h, plan->params.trace, sizeof(h), cudaMemcpyDeviceToHost);
      const long long t0 = h[0];
      const GemmParams& p = plan->params;
      std::fprintf(stderr, "trace: BN %d BK %d group %d stages %d num_kb %d m_tiles %d n_tiles %d grid %d conv %d span %d\n", p.BN, p.BK,
                   p.group, p.stages, p.num_kb, p.m_tiles, p.n_tiles, plan->grid, p.conv, p.store_span);
      std::fprintf(stderr, "marks: entry %lld  prologue done %lld  all roles done %lld (cycles from first producer wait)\n", h[384] - t0, h[385] - t0, h[386] - t0);
      for (int i = 0; i < 20; ++i)
        std::fprintf(stderr, "it %2d  prodA slot-free %7lld issued %7lld | mma data-in %7lld committed %7lld | epi acc-ready %7lld done %7lld\n",
                     i, h[(0 * 64 + i) * 2] - t0, h[(0 * 64 + i) * 2 + 1] - t0, h[(1 * 64 + i) * 2] - t0,
                     h[(1 * 64 + i) * 2 + 1] - t0, h[(2 * 64 + i) * 2] - t0, h[(2 * 64 + i) * 2 + 1] - t0);
      for (int i = 0; i < 12; ++i)
        std::fprintf(stderr, "epi warp %d tile %2d  top %7lld accumulator ready %7lld residual ready %7lld chunks done %7lld\n", B2VX_TRACE_WARP, i,
                     h[400 + i * 8] - t0, h[400 + i * 8 + 1] - t0, h[400 + i * 8 + 2] - t0, h[400 + i * 8 + 3] - t0);
    }
  }
#endif
  return cudaGetLastError();
}

}  // namespace b2vx
