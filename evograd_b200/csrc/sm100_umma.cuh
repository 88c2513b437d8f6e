// Inline-PTX building blocks for Blackwell (sm_100a) tensor-core kernels:
// mbarriers with bounded waits, TMA tile loads, tensor-memory (TMEM) allocation
// and access, tcgen05.mma issue with shared-memory / TMEM operands.
//
// Every wait in this file gives up after a cycle budget and records the fact
// in an abort word, after which all later waits return immediately, so a kernel
// built from these pieces always runs to its end, frees its TMEM and returns.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace evg {
namespace umma {

// ------------------------------------------------------------------ host side
// Encodes a TMA descriptor for a dense [outer, rows, cols] tensor of 16-bit
// elements (fmt 0 = float16, 1 = bfloat16) whose tiles are [box_rows x 64] with
// the 128-byte swizzle that the tcgen05 shared-memory descriptors below expect.
// Returns false on failure.
bool encode_tile_map_16bit(CUtensorMap* map, const void* base, int fmt, uint64_t cols,
                           uint64_t rows, uint64_t outer, uint32_t box_rows);

// A 16-bit [B, H, S, D] tensor (token_major: [B, S, H, D]) as a 4-D map with
// coordinates (column, position, head, batch) and the same [box_rows x 64] tiles.
bool encode_tile_map_16bit_4d(CUtensorMap* map, const void* base, int fmt, uint64_t D, uint64_t S,
                              uint64_t H, uint64_t B, uint32_t box_rows, bool token_major);

// The same for a dense float32 [outer, rows, cols] tensor with tiles of
// [box_rows x box_cols]; swizzle128 needs box_cols == 32 (128 bytes per row).
bool encode_tile_map_f32(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows,
                         uint64_t outer, uint32_t box_cols, uint32_t box_rows, bool swizzle128);

#ifdef __CUDACC__
// ---------------------------------------------------------------- device side

constexpr uint32_t kAtomBytesPerRow = 128;  // one swizzle atom row: 64 x 16-bit
constexpr uint32_t kAtomGroupBytes = 1024;  // 8 rows of an atom

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// Abort protocol shared by all waits of a block.
struct WaitCtx {
  volatile int* abort_flag;   // shared memory word, 0 until a wait times out
  int* device_status;         // global sticky status word
  long long limit_cycles;
};

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity to complete, at most
// ctx.limit_cycles; on timeout sets the abort word (code identifies the wait).
// Returns false when the wait was given up (now, or by an earlier wait of the
// block), true when the phase completed.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx,
                                          int code) {
  // Fast path first: a phase that has already completed costs one try_wait and no
  // shared-memory load (the abort word only matters while actually waiting).
  if (mbar_try_wait(bar, parity)) return true;
  if (*ctx.abort_flag) return false;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*ctx.abort_flag) return false;
    if (clock64() - start > ctx.limit_cycles) {
      *ctx.abort_flag = code;
      atomicCAS(ctx.device_status, 0, code);
      return false;
    }
  }
  return true;
}

// After an abort the producer stops issuing copies; the ones already issued
// still write into this block's shared memory, which the next block resident on
// the SM may reuse. The issuing thread therefore lets them land (a bounded wait
// that ignores the abort word and records nothing) before the block returns.
__device__ __forceinline__ void mbar_drain(uint64_t* bar, uint32_t parity, long long limit_cycles) {
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity))
    if (clock64() - start > limit_cycles) return;
}
// For kernels whose hot loop cannot afford to track what it has issued (one
// more live register per row costs the norm backward 3 % of its time): after a
// timeout the issuing thread simply gives the bulk copies still in flight time
// to land (a copy completes in a few microseconds; this waits a hundred) before
// the block and its shared memory are given up.
__device__ __forceinline__ void settle_after_abort() {
  const long long start = clock64();
  while (clock64() - start < (1ll << 18)) {
  }
}

// TMA: global -> shared tile load, completion counted on an mbarrier.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int c0, int c1,
                                            int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, int c0, int c1,
                                            int c2, int c3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a
// multiple of 16 bytes), completion counted on an mbarrier. No multicast.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// Tensor memory. alloc/dealloc/relinquish are warp-collective.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp gets lane (base+i),
// register j is column (col+j).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}

// 32 lanes x 16 columns.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 8 columns.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// The same accesses chosen by the width of the register array.
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t (&r)[16]) { tmem_st16(taddr, r); }
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t (&r)[8]) { tmem_st8(taddr, r); }

// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).
// Field layout: start address [0,14), leading byte offset [16,30), stride byte
// offset [32,46) (all in 16-byte units), version [46,48), layout type [61,64).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// A tile is stored as [cols/64] swizzle-atom columns, each [rows x 64] 16-bit
// elements (rows * 128 bytes), 1024-byte aligned.
//
// K-major use (the contraction runs along the tile's columns): k-step `ks`
// (16 elements) lives in atom column ks/4 at byte offset (ks%4)*32; 8-row
// groups are 1024 bytes apart; the leading offset is unused for swizzled
// K-major operands and is set to the conventional 1.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_saddr, uint32_t rows, int ks) {
  const uint32_t addr = tile_saddr + (uint32_t)(ks >> 2) * rows * kAtomBytesPerRow + (ks & 3) * 32;
  return smem_desc_sw128(addr, 16, kAtomGroupBytes);
}
// MN-major use (the contraction runs along the tile's ROWS, the columns are the
// operand's M/N extent): k-step `ks` covers rows [16ks, 16ks+16); the next 64
// columns are one atom column (rows*128 bytes) further on; 8-row groups are
// 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_saddr, uint32_t rows, int ks) {
  const uint32_t addr = tile_saddr + (uint32_t)ks * 16 * kAtomBytesPerRow;
  return smem_desc_sw128(addr, rows * kAtomBytesPerRow, kAtomGroupBytes);
}

// The same descriptors split into a per-tile base and a per-k-step increment, so
// that the single issuing thread spends one integer add per operand per MMA
// (building a descriptor from scratch costs more issue cycles than the MMA takes
// to execute). The start-address field holds (address >> 4) in 14 bits; shared
// memory is < 256 KB, so adding a k-step offset never carries out of the field.
struct DescBase {
  uint32_t lo;  // start address | leading byte offset
  uint32_t hi;  // stride byte offset | version | swizzle mode
};
__device__ __forceinline__ DescBase desc_base_kmajor(uint32_t tile_saddr) {
  return DescBase{((tile_saddr & 0x3FFFFu) >> 4) | (1u << 16),
                  (kAtomGroupBytes >> 4) | (1u << 14) | (2u << 29)};
}
__device__ __forceinline__ DescBase desc_base_mnmajor(uint32_t tile_saddr, uint32_t rows) {
  return DescBase{((tile_saddr & 0x3FFFFu) >> 4) | (((rows * kAtomBytesPerRow) >> 4) << 16),
                  (kAtomGroupBytes >> 4) | (1u << 14) | (2u << 29)};
}
// k-step increments of the start-address field (units of 16 bytes).
__host__ __device__ constexpr uint32_t kstep_kmajor(uint32_t rows, int ks) {
  return ((uint32_t)(ks >> 2) * rows * kAtomBytesPerRow + (uint32_t)(ks & 3) * 32u) >> 4;
}
__host__ __device__ constexpr uint32_t kstep_mnmajor(int ks) {
  return ((uint32_t)ks * 16u * kAtomBytesPerRow) >> 4;
}
__device__ __forceinline__ uint64_t desc_at(const DescBase& b, uint32_t step) {
  return ((uint64_t)b.hi << 32) | (uint64_t)(b.lo + step);
}

// Instruction descriptor for kind::f16 with float32 accumulation.
// fmt: 0 = f16, 1 = bf16. *_mn: 1 when that operand is MN-major.
__host__ __device__ constexpr uint32_t instr_desc_f16(int fmt, int m, int n, int a_mn, int b_mn) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)a_mn << 15) |
         ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// 2^x on the special-function unit, denormals flushed (inputs here are scores
// minus a log-sum-exp: anything that small is zero after rounding to 16 bits).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One lane of a converged warp (warp-collective). The issuing warp runs its
// whole program on all 32 lanes and predicates only the tcgen05 instruction
// with this, so that descriptors and addresses stay warp-uniform values (the
// instruction takes them from uniform registers; computing them inside a
// divergent single-lane branch forces per-operand transfers that cost more
// issue time than the MMA takes to execute).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A holds two 16-bit elements per 32-bit column.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Makes `bar` complete one arrival when every MMA issued so far by this thread
// has finished (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

#endif  // __CUDACC__
}  // namespace umma
}  // namespace evg
