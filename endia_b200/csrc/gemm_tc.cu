// fp32 GEMM on the 5th-generation tensor cores (tcgen05) with split-precision products:
//   a = a_hi + a_lo,  a_hi = a with the 13 low mantissa bits cleared (exactly a tf32 value; the
//   tensor core reads fp32 storage that way, so the raw array is the hi operand),
//   a*b ~= a_hi*b_hi + a_lo*b + a*b_lo              (fp32 accumulation in tensor memory)
// 3xTF32 forms all three products with tf32 MMAs on fp32 low parts (~21 bits per product); the
// bf16-compensated scheme forms the two corrections with bf16 MMAs on bf16(a_lo), bf16(b), bf16(a),
// bf16(b_lo) (~19 bits per product, two thirds of the tensor-core time). Either way gradients stay
// within 1e-4 of the fp32 result; plain tf32 (one product) is never used.
//
// Two kernels:
//   gemm_tc2p_kernel  persistent, clusters of two CTAs (cta_group::2, 256 x 256 tiles), both
//                     schemes, bulk-tensor-store epilogue, optional two-way K split (N >= 256)
//   gemm_tc_kernel    one CTA per 128 x BN tile, 3xTF32, optional split-K over blockIdx.y
// Structure of a CTA (320 threads):
//   warp 0   : producer - one lane issues TMA tile loads (the fp32 tile and the operand parts of A
//              and B, swizzled) into a ring of shared-memory stages, signalled through mbarriers
//   warp 1   : allocates tensor memory (two accumulators of BN columns: the hi*hi sum and the
//              sum of the two correction products); one lane issues tcgen05.mma and commits each
//              stage back to the producer
//   warps 2-9: epilogue - tcgen05.ld of the accumulators (one row per thread, two warps per lane
//              quarter, each half of the columns), their sum through a swizzled shared-memory
//              chunk, the fused epilogue of endia_b200_epilogue with eight lanes along a row, and
//              the store (bulk tensor store in the persistent kernel, 128-bit stores otherwise)
// Operands are consumed in the layout they have in global memory: a row-major [rows, K] operand
// is K-major, a stored-transposed one ([K, rows]) is MN-major, selected in the instruction and
// shared-memory descriptors, so dX = dY*W^T and dW = X^T*dY need no transposed copies
// (endia/functional/binary_ops/matmul_op.mojo:107-136, 278-284).
// Every wait on an mbarrier is bounded; a wait that gives up records a code in a device flag
// (endia_b200_device_status) and the CTA drains and returns.
#include "common.cuh"
#include "gemm.cuh"
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdlib.h>

namespace eb {

constexpr int TC_BM = 128;
constexpr int TC_GROUP_M = 8;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 22;

static __device__ int g_tc_status = 0;    // 0 ok, else the code of the first wait that gave up


// ------------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false (and the status flag set) when the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code,
                                          uint32_t limit = TC_WAIT_LIMIT) {
  for (uint32_t it = 0; it < limit; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  atomicCAS(&g_tc_status, 0, code);
  return false;
}

// Self-test of the give-up path: one thread waits, with the wait above and a limit of `polls`, on a
// barrier that nothing ever arrives at. The wait runs out, records code 99 and the kernel returns.
__global__ void wait_selftest_kernel(uint32_t polls) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait(smem_u32(&bar), 0, 99, polls);
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (descriptor version 1): start address, leading and stride byte
// offsets in 16-byte units, and the swizzle mode: 2 = 128-byte swizzle in 16-byte units (K-major
// tiles), 1 = 128-byte swizzle in 32-byte units, the only mode MN-major 32-bit operands accept.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)layout_type << 61;
  return d;
}
// K-major tile: rows of BK floats (128 bytes with the 128-byte swizzle, 64 with the 64-byte one),
// 8-row groups contiguous. MN-major tile: boxes of [BK k][32 rows] (BK*128 bytes apart), inside
// a box groups of 4 k-rows 512 bytes apart.
template <bool MN_MAJOR, int BK>
__device__ __forceinline__ uint64_t tile_desc(uint32_t addr) {
  return MN_MAJOR ? smem_desc(addr, BK * 128, 512, 1)
                  : smem_desc(addr, 16, 8 * BK * 4, BK == 32 ? 2 : 4);
}

struct TcMaps {
  CUtensorMap a_hi, a_lo, b_hi, b_lo;
  CUtensorMap a16h, a16l, b16h, b16l;   // bf16 parts of the operands (bf16-compensated scheme)
  CUtensorMap c;   // output, boxes of [32 rows][32 floats] (persistent kernel, when C allows 128-bit access)
};

// Bulk tensor store of one [32 rows][128 bytes] shared-memory box (128-byte swizzle) to C at
// column x, row y; rows and columns beyond the array are clipped by the copy engine.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
// The same box added (fp32) to what C holds.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ float4 lds128(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t a, float4 v) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// The fused epilogue on four consecutive columns n..n+3 of row m; `vec` says that the bias, the
// activation-derivative source and C may be read with 128-bit loads at this position.
__device__ __forceinline__ float4 apply_epilogue4(const EpiParams &e, float4 acc, int64_t m, int64_t n,
                                                  const float *c_old, bool vec) {
  if (!vec) {
    float4 o;
    o.x = apply_epilogue(e, acc.x, m, n + 0, c_old + 0);
    o.y = apply_epilogue(e, acc.y, m, n + 1, c_old + 1);
    o.z = apply_epilogue(e, acc.z, m, n + 2, c_old + 2);
    o.w = apply_epilogue(e, acc.w, m, n + 3, c_old + 3);
    return o;
  }
  float4 v = make_float4(e.alpha * acc.x, e.alpha * acc.y, e.alpha * acc.z, e.alpha * acc.w);
  if (e.bias) {
    const float4 b = __ldg(reinterpret_cast<const float4 *>(e.bias + n));
    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
  }
  if (e.act) { v.x = act_fwd(e.act, v.x); v.y = act_fwd(e.act, v.y); v.z = act_fwd(e.act, v.z); v.w = act_fwd(e.act, v.w); }
  if (e.dact) {
    const float4 d = __ldg(reinterpret_cast<const float4 *>(e.dact_src + m * e.ld_dact + n));
    v.x *= act_bwd(e.dact, d.x); v.y *= act_bwd(e.dact, d.y); v.z *= act_bwd(e.dact, d.z); v.w *= act_bwd(e.dact, d.w);
  }
  if (e.beta != 0.f) {
    const float4 c = *reinterpret_cast<const float4 *>(c_old);
    v.x += e.beta * c.x; v.y += e.beta * c.y; v.z += e.beta * c.z; v.w += e.beta * c.w;
  }
  return v;
}

// Epilogue of one warp: rows of tensor-memory lane quarter q, column chunks [c_begin, c_end) of
// 32 columns each. tcgen05.ld hands each thread one ROW of the chunk; storing that directly would
// touch 32 different rows per instruction. So the sum of the two accumulators goes through a
// [32 rows][128 bytes] shared-memory buffer (16-byte units XOR-swizzled with the row, two buffers
// per warp at `buf`, taken from the operand stages that are free by now) and is read back with
// eight lanes along each row: every global access of the fused epilogue (C, the activation
// source, the bias) then covers whole 128-byte lines. The tensor-memory loads of the next chunk
// are in flight while a chunk is processed.
template <int BN, bool DOUBLE_BUF = true>
__device__ __forceinline__ void tc_epilogue_warp(uint32_t tmem_base, int q, int lane, int c_begin, int c_end,
                                                 int64_t m0, int64_t n0, int64_t M, int64_t N, float *Cout,
                                                 int64_t ldc, const EpiParams &epi, bool vec_c, uint32_t buf) {
  const uint32_t row_addr = tmem_base + ((uint32_t)(q * 32) << 16);
  const bool vec_epi = vec_c && (!epi.bias || (reinterpret_cast<uintptr_t>(epi.bias) & 15) == 0) &&
                       (!epi.dact || ((reinterpret_cast<uintptr_t>(epi.dact_src) & 15) == 0 && epi.ld_dact % 4 == 0));
  uint32_t ra[32], rb[32];
  const int c4 = lane & 7, rsub = lane >> 3;
  tc_ld32(row_addr + (uint32_t)(c_begin * 32), ra);
  tc_ld32(row_addr + (uint32_t)(BN + c_begin * 32), rb);
#pragma unroll 1
  for (int c = c_begin; c < c_end; ++c) {
    const uint32_t bb = buf + (DOUBLE_BUF ? (uint32_t)(c & 1) * 4096u : 0u);
    tc_wait_ld();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float4 v;
      v.x = __uint_as_float(ra[4 * j + 0]) + __uint_as_float(rb[4 * j + 0]);
      v.y = __uint_as_float(ra[4 * j + 1]) + __uint_as_float(rb[4 * j + 1]);
      v.z = __uint_as_float(ra[4 * j + 2]) + __uint_as_float(rb[4 * j + 2]);
      v.w = __uint_as_float(ra[4 * j + 3]) + __uint_as_float(rb[4 * j + 3]);
      sts128(bb + (uint32_t)lane * 128u + (uint32_t)((j ^ (lane & 7)) * 16), v);
    }
    if (c + 1 < c_end) {   // in flight while this chunk goes out to global memory
      tc_ld32(row_addr + (uint32_t)((c + 1) * 32), ra);
      tc_ld32(row_addr + (uint32_t)(BN + (c + 1) * 32), rb);
    }
    __syncwarp();
    const int64_t n = n0 + c * 32 + c4 * 4;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = rsub + 4 * i;
      const int64_t m = m0 + q * 32 + r;
      const float4 v = lds128(bb + (uint32_t)r * 128u + (uint32_t)((c4 ^ (r & 7)) * 16));
      if (m >= M || n >= N) continue;
      float *cp = Cout + m * ldc + n;
      if (vec_c && n + 4 <= N) {
        *reinterpret_cast<float4 *>(cp) = apply_epilogue4(epi, v, m, n, cp, vec_epi);
      } else {
        const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int t = 0; t < 4; ++t)
          if (n + t < N) cp[t] = apply_epilogue(epi, e[t], m, n + t, cp + t);
      }
    }
    if (!DOUBLE_BUF) __syncwarp();   // the buffer is rewritten by the next chunk
  }
}

// ------------------------------------------------------------------------------------ kernel
// A_MN / B_MN: the operand is MN-major in global memory (stored [K, rows]); its tile then arrives
// as rows/32 boxes of [BK k][32 rows].
template <int BN, int BK, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(320, 1)
gemm_tc_kernel(const __grid_constant__ TcMaps maps, const GemmParams p, int tiles_m) {
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr uint32_t A_BYTES = TC_BM * BK * 4;
  constexpr uint32_t B_BYTES = BN * BK * 4;
  constexpr uint32_t BOX_BYTES = BK * 128;          // one [BK k][32 rows] box of an MN-major tile
  constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  const uint32_t smem_base = (smem_u32(smem) + 1023u) & ~1023u;
  const uint32_t bars = smem_base + STAGES * STAGE_BYTES;   // full[STAGES], empty[STAGES], acc
  __shared__ uint32_t tmem_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_m = blockIdx.x % tiles_m, tile_n = blockIdx.x / tiles_m;
  const int m0 = tile_m * TC_BM, n0 = tile_n * BN;
  // split-K: blockIdx.y takes one contiguous range of k-blocks and writes raw sums to its slice
  // of p.partial; a second kernel adds the slices in order and applies the epilogue.
  const int splits = gridDim.y;
  const int nkb_total = (int)((p.K + BK - 1) / BK);
  const int kb_per = (nkb_total + splits - 1) / splits;
  const int kb0 = blockIdx.y * kb_per;
  int nkb = nkb_total - kb0;
  nkb = nkb < 0 ? 0 : (nkb > kb_per ? kb_per : nkb);
  float *Cout = p.C;
  int64_t ldc = p.ldc;
  EpiParams epi = p.epi;
  bool vec_c = p.vec_c;
  if (splits > 1) {
    Cout = p.partial + (int64_t)blockIdx.y * p.M * p.ld_partial;
    ldc = p.ld_partial;
    epi = EpiParams{1.f, 0.f, nullptr, 0, 0, nullptr, 0, nullptr};
    vec_c = true;
  }
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t acc_bar = bars + 8u * (2 * STAGES);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)(2 * BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % STAGES;
        if (kb >= STAGES) ok = mbar_wait(empty_bar(s), ((kb / STAGES) - 1) & 1, 1);
        if (!ok) break;
        const uint32_t st = smem_base + s * STAGE_BYTES;
        const uint32_t fb = full_bar(s);
        mbar_expect_tx(fb, STAGE_BYTES);
        const int k0 = (kb0 + kb) * BK;
        if constexpr (A_MN) {
#pragma unroll
          for (int j = 0; j < TC_BM / 32; ++j) {
            tma_load_2d(st + j * BOX_BYTES, &maps.a_hi, fb, m0 + 32 * j, k0);
            tma_load_2d(st + A_BYTES + j * BOX_BYTES, &maps.a_lo, fb, m0 + 32 * j, k0);
          }
        } else {
          tma_load_2d(st, &maps.a_hi, fb, k0, m0);
          tma_load_2d(st + A_BYTES, &maps.a_lo, fb, k0, m0);
        }
        const uint32_t sb = st + 2 * A_BYTES;
        if constexpr (B_MN) {
#pragma unroll
          for (int j = 0; j < BN / 32; ++j) {
            tma_load_2d(sb + j * BOX_BYTES, &maps.b_hi, fb, n0 + 32 * j, k0);
            tma_load_2d(sb + B_BYTES + j * BOX_BYTES, &maps.b_lo, fb, n0 + 32 * j, k0);
          }
        } else {
          tma_load_2d(sb, &maps.b_hi, fb, k0, n0);
          tma_load_2d(sb + B_BYTES, &maps.b_lo, fb, k0, n0);
        }
        ++issued;
      }
      if (!ok) {
        // Give copies already in flight a bounded chance to land before the CTA exits.
        for (int kb = (issued > STAGES ? issued - STAGES : 0); kb < issued; ++kb)
          mbar_wait(full_bar(kb % STAGES), (kb / STAGES) & 1, 2);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // Instruction descriptor: fp32 accumulator, tf32 A and B, majors, N >> 3, M >> 4.
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) |
                             ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(TC_BM >> 4) << 24);
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % STAGES;
        ok = mbar_wait(full_bar(s), (kb / STAGES) & 1, 3);
        if (!ok) break;
        tc_fence_after();
        const uint32_t st = smem_base + s * STAGE_BYTES;
        const uint64_t a_hi = tile_desc<A_MN, BK>(st), a_lo = tile_desc<A_MN, BK>(st + A_BYTES);
        const uint32_t sb = st + 2 * A_BYTES;
        const uint64_t b_hi = tile_desc<B_MN, BK>(sb), b_lo = tile_desc<B_MN, BK>(sb + B_BYTES);
        // One k-step (K = 8 floats) further: 32 bytes along a K-major row, one 8-row (1024-byte)
        // block of an MN-major tile; in 16-byte descriptor units.
        constexpr uint64_t A_STEP = A_MN ? 64 : 2, B_STEP = B_MN ? 64 : 2;
#pragma unroll
        for (int ks = 0; ks < BK / 8; ++ks) {
          const uint64_t ah = a_hi + ks * A_STEP, al = a_lo + ks * A_STEP;
          const uint64_t bh = b_hi + ks * B_STEP, bl = b_lo + ks * B_STEP;
          // The two correction products accumulate in their own tensor-memory columns: the
          // accumulator adds round toward zero, so every add into the large sum costs up to one
          // ulp of it, and keeping the small terms apart leaves one such add per k-step.
          const uint32_t acc = (kb | ks) ? 1u : 0u;
          tc_mma_tf32(tmem_base + BN, al, bh, idesc, acc);
          tc_mma_tf32(tmem_base + BN, ah, bl, idesc, 1u);
          tc_mma_tf32(tmem_base, ah, bh, idesc, acc);
        }
        tc_commit(empty_bar(s));   // frees the stage once these MMAs have read it
      }
      tc_commit(acc_bar);          // accumulator complete (also on the give-up path)
    }
  } else {
    // --------------------------------------------------------------------- epilogue
    const int q = warp & 3;        // tensor-memory lane quarter this warp may read
    const int half = (warp - 2) >> 2;   // warps 2-5 take the first half of the columns, 6-9 the second
    const bool ok = mbar_wait(acc_bar, 0, 4);
    tc_fence_after();
    const int64_t m = (int64_t)m0 + q * 32 + lane;
    if (ok && nkb > 0) {
      constexpr int CH = BN / 64;
      tc_epilogue_warp<BN>(tmem_base, q, lane, half * CH, (half + 1) * CH, m0, n0, p.M, p.N, Cout, ldc, epi, vec_c,
                           smem_base + (uint32_t)(warp - 2) * 8192u);
    } else if (ok && m < p.M && half == 0) {
      // K == 0: the product is empty, the epilogue applies to zeros.
      for (int64_t n = n0; n < n0 + BN && n < p.N; ++n)
        Cout[m * ldc + n] = apply_epilogue(epi, 0.f, m, n, Cout + m * ldc + n);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * BN)) : "memory");
  }
}

// ------------------------------------------------------------- two-CTA (cta_group::2) kernel
// A pair of CTAs on neighbouring SMs computes one 256 x 256 tile: each CTA keeps its own 128 rows
// of A and only HALF of the B tile in shared memory; the leader CTA issues tcgen05.mma with
// cta_group::2 (M = 256), which reads both halves of B and writes each CTA's 128 accumulator rows
// into that CTA's tensor memory. Per CTA this halves the B traffic into and out of shared
// memory, the resource that bounds the one-CTA kernel. Loads of both CTAs signal the leader's
// "full" barriers; the leader's commits are multicast to both CTAs' "empty" and accumulator
// barriers. No load is multicast.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Tile load whose completion bytes are counted on a barrier of the pair's leader CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t leader_bar,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// bf16 tiles of 32 k: K-major rows of 64 bytes (64-byte swizzle, 8-row groups 512 bytes apart);
// MN-major boxes of [32 k][64 rows] (128 bytes per k-row, 128-byte swizzle, 8 k-rows per atom,
// boxes 4096 bytes apart).
template <bool MN_MAJOR>
__device__ __forceinline__ uint64_t tile_desc16(uint32_t addr) {
  return MN_MAJOR ? smem_desc(addr, 4096, 1024, 2) : smem_desc(addr, 16, 512, 4);
}

// Epilogue of one warp of the persistent kernel, in two steps. tc_epilogue_drain moves the warp's
// 32 rows x 128 columns (the sum of the two accumulators) from tensor memory into registers; the
// caller then hands the accumulators back to the MMA issuer, so that the next tile's products run
// while tc_epilogue_warp_bulk finishes this one: chunk by chunk of [32 x 32] through the warp's
// shared-memory buffer and out with a bulk tensor store issued by one lane (the register path of
// 128-bit stores drains a tile several times slower). The fused epilogue runs in place on the
// shared-memory chunk with eight lanes along each row, so that its reads of the activation
// source, the bias and C are coalesced; a plain product skips that pass.
// with_corr = false: a run before the last one: the correction accumulator keeps running (its
// truncation is 2^-11 of the main one's) and only the main accumulator is drained.
__device__ __forceinline__ void tc_stage_chunk(uint32_t buf, int lane, const uint32_t (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float4 x = make_float4(__uint_as_float(v[4 * j + 0]), __uint_as_float(v[4 * j + 1]),
                                 __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
    sts128(buf + (uint32_t)lane * 128u + (uint32_t)((j ^ (lane & 7)) * 16), x);
  }
}

// (the first chunk goes straight to the warp's shared-memory buffer, the other three stay in
// registers: 96 values per lane)
template <int BN>
__device__ __forceinline__ void tc_epilogue_drain(uint32_t tmem_base, int q, int lane, int c_begin, bool with_corr,
                                                  uint32_t buf, uint32_t (&v1)[32], uint32_t (&v2)[32],
                                                  uint32_t (&v3)[32]) {
  const uint32_t row_addr = tmem_base + ((uint32_t)(q * 32) << 16);
  uint32_t rb[16];
#define EB_ADD_CORR(C, V)                                                                  \
  if (with_corr) {                                                                         \
    _Pragma("unroll") for (int h = 0; h < 2; ++h) {                                        \
      tc_ld16(row_addr + (uint32_t)(BN + (c_begin + C) * 32 + 16 * h), rb);                \
      tc_wait_ld();                                                                        \
      _Pragma("unroll") for (int j = 0; j < 16; ++j)                                       \
        V[16 * h + j] = __float_as_uint(__uint_as_float(V[16 * h + j]) + __uint_as_float(rb[j])); \
    }                                                                                      \
  }
  {
    uint32_t v0[32];
    tc_ld32(row_addr + (uint32_t)((c_begin + 0) * 32), v0);
    // the last store of the previous tile has read the buffer
    if (lane == 0) bulk_wait_read0();
    __syncwarp();
    tc_wait_ld();
    EB_ADD_CORR(0, v0)
    tc_stage_chunk(buf, lane, v0);
  }
  tc_ld32(row_addr + (uint32_t)((c_begin + 1) * 32), v1);
  tc_ld32(row_addr + (uint32_t)((c_begin + 2) * 32), v2);
  tc_ld32(row_addr + (uint32_t)((c_begin + 3) * 32), v3);
  tc_wait_ld();
  EB_ADD_CORR(1, v1)
  EB_ADD_CORR(2, v2)
  EB_ADD_CORR(3, v3)
#undef EB_ADD_CORR
}

__device__ __forceinline__ void tc_epilogue_warp_bulk(const uint32_t (&v1)[32], const uint32_t (&v2)[32],
                                                      const uint32_t (&v3)[32], int q,
                                                      int lane, int c_begin, int64_t m0, int64_t n0, int64_t M,
                                                      int64_t N, const float *Cout, int64_t ldc,
                                                      const EpiParams &epi, const CUtensorMap *cmap, uint32_t buf,
                                                      bool reduce, bool raw, bool pre_add, int64_t row_off) {
  // row_off: added to the row coordinate of the stores (the slice of a split-K work buffer).
  // raw: this is a partial run of a reduction whose epilogue is not linear: the bare sums are
  // stored (or added); pre_add: the last run of such a reduction, which adds what the earlier runs
  // left in C before it applies the epilogue.
  const bool plain = raw || (epi.alpha == 1.f && !epi.bias && !epi.act && !epi.dact && epi.beta == 0.f &&
                             !epi.colsum_partial && !pre_add && !epi.c16);
  const bool vec_epi = (!epi.bias || (reinterpret_cast<uintptr_t>(epi.bias) & 15) == 0) &&
                       (!epi.dact || ((reinterpret_cast<uintptr_t>(epi.dact_src) & 15) == 0 && epi.ld_dact % 4 == 0));
  const int c4 = lane & 7, rsub = lane >> 3;
#pragma unroll 1
  for (int ci = 0; ci < 4; ++ci) {
    const int c = c_begin + ci;
    if (ci > 0) {   // (chunk 0 was staged by tc_epilogue_drain)
      // the previous chunk's store has read the buffer
      if (lane == 0) bulk_wait_read0();
      __syncwarp();
      switch (ci) {
        case 1: tc_stage_chunk(buf, lane, v1); break;
        case 2: tc_stage_chunk(buf, lane, v2); break;
        default: tc_stage_chunk(buf, lane, v3); break;
      }
    }
    const int64_t nb = n0 + c * 32;
    if (!plain) {
      __syncwarp();
      const int64_t n = nb + c4 * 4;
      float4 cs = make_float4(0.f, 0.f, 0.f, 0.f);   // column sums of this lane's 8 rows
      if (vec_epi && epi.beta == 0.f && m0 + q * 32 + 32 <= M && nb + 32 <= N) {
        // a chunk inside the matrix (all of them but the ragged edges): the same steps on whole
        // float4s, with everything that does not depend on the row taken out of the loop
        const float alpha = epi.alpha;
        const int act = epi.act, dact = epi.dact;
        const float4 b4 = epi.bias ? __ldg(reinterpret_cast<const float4 *>(epi.bias + n)) : make_float4(0.f, 0.f, 0.f, 0.f);
        const int64_t mr = m0 + q * 32 + rsub;
        const float *cp = Cout + mr * ldc + n;
        const float *dp = dact ? epi.dact_src + mr * epi.ld_dact + n : nullptr;
        __nv_bfloat16 *h16 = epi.c16 ? static_cast<__nv_bfloat16 *>(epi.c16) + mr * ldc + n : nullptr;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = rsub + 4 * i;
          const uint32_t a = buf + (uint32_t)r * 128u + (uint32_t)((c4 ^ (r & 7)) * 16);
          float4 v = lds128(a);
          if (pre_add) {
            const float4 c = __ldcg(reinterpret_cast<const float4 *>(cp + (int64_t)(4 * i) * ldc));
            v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
          }
          v.x = alpha * v.x + b4.x; v.y = alpha * v.y + b4.y; v.z = alpha * v.z + b4.z; v.w = alpha * v.w + b4.w;
          if (act) { v.x = act_fwd(act, v.x); v.y = act_fwd(act, v.y); v.z = act_fwd(act, v.z); v.w = act_fwd(act, v.w); }
          if (dact) {
            const float4 d = __ldg(reinterpret_cast<const float4 *>(dp + (int64_t)(4 * i) * epi.ld_dact));
            v.x *= act_bwd(dact, d.x); v.y *= act_bwd(dact, d.y); v.z *= act_bwd(dact, d.z); v.w *= act_bwd(dact, d.w);
          }
          cs.x += v.x; cs.y += v.y; cs.z += v.z; cs.w += v.w;
          sts128(a, v);
          if (h16) {
            // the operand parts of the stored values, for the products that will read C
            const __nv_bfloat162 h01 = __floats2bfloat162_rn(v.x, v.y), h23 = __floats2bfloat162_rn(v.z, v.w);
            const __nv_bfloat162 l01 = __floats2bfloat162_rn(v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u),
                                                             v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u));
            const __nv_bfloat162 l23 = __floats2bfloat162_rn(v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u),
                                                             v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u));
            uint2 hv, lv;
            hv.x = *reinterpret_cast<const uint32_t *>(&h01); hv.y = *reinterpret_cast<const uint32_t *>(&h23);
            lv.x = *reinterpret_cast<const uint32_t *>(&l01); lv.y = *reinterpret_cast<const uint32_t *>(&l23);
            __nv_bfloat16 *hp = h16 + (int64_t)(4 * i) * ldc;
            *reinterpret_cast<uint2 *>(hp) = hv;
            *reinterpret_cast<uint2 *>(hp + epi.c16_lo) = lv;
          }
        }
      } else
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = rsub + 4 * i;
        const int64_t m = m0 + q * 32 + r;
        const uint32_t a = buf + (uint32_t)r * 128u + (uint32_t)((c4 ^ (r & 7)) * 16);
        if (m >= M || n >= N) continue;
        float4 v = lds128(a);
        const float *cp = Cout + m * ldc + n;
        if (n + 4 <= N) {
          if (pre_add) {
            const float4 c = __ldcg(reinterpret_cast<const float4 *>(cp));
            v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
          }
          v = apply_epilogue4(epi, v, m, n, cp, vec_epi);
        } else {
          float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int t = 0; t < 4; ++t)
            e[t] = (n + t < N) ? apply_epilogue(epi, e[t] + (pre_add ? __ldcg(cp + t) : 0.f), m, n + t, cp + t) : 0.f;
          v = make_float4(e[0], e[1], e[2], e[3]);
        }
        cs.x += v.x; cs.y += v.y; cs.z += v.z; cs.w += v.w;
        sts128(a, v);
        if (epi.c16) {
          // the operand parts of the stored values, for the products that will read C
          __nv_bfloat16 *h16 = static_cast<__nv_bfloat16 *>(epi.c16) + m * ldc + n, *l16 = h16 + epi.c16_lo;
          const float e[4] = {v.x, v.y, v.z, v.w};
          if (n + 4 <= N) {
            const __nv_bfloat162 h01 = __floats2bfloat162_rn(e[0], e[1]), h23 = __floats2bfloat162_rn(e[2], e[3]);
            const __nv_bfloat162 l01 = __floats2bfloat162_rn(e[0] - __uint_as_float(__float_as_uint(e[0]) & 0xFFFFE000u),
                                                             e[1] - __uint_as_float(__float_as_uint(e[1]) & 0xFFFFE000u));
            const __nv_bfloat162 l23 = __floats2bfloat162_rn(e[2] - __uint_as_float(__float_as_uint(e[2]) & 0xFFFFE000u),
                                                             e[3] - __uint_as_float(__float_as_uint(e[3]) & 0xFFFFE000u));
            uint2 hv, lv;
            hv.x = *reinterpret_cast<const uint32_t *>(&h01); hv.y = *reinterpret_cast<const uint32_t *>(&h23);
            lv.x = *reinterpret_cast<const uint32_t *>(&l01); lv.y = *reinterpret_cast<const uint32_t *>(&l23);
            *reinterpret_cast<uint2 *>(h16) = hv;
            *reinterpret_cast<uint2 *>(l16) = lv;
          } else {
#pragma unroll
            for (int t = 0; t < 4; ++t)
              if (n + t < N) {
                h16[t] = __float2bfloat16_rn(e[t]);
                l16[t] = __float2bfloat16_rn(e[t] - __uint_as_float(__float_as_uint(e[t]) & 0xFFFFE000u));
              }
          }
        }
      }
      if (epi.colsum_partial) {
        // the bias gradient: sum over the warp's 32 rows (the four lanes that share c4), one
        // partial row per 32 rows of C, added up in a fixed order by colsum_finish_kernel
        cs.x += __shfl_xor_sync(0xffffffffu, cs.x, 8);  cs.y += __shfl_xor_sync(0xffffffffu, cs.y, 8);
        cs.z += __shfl_xor_sync(0xffffffffu, cs.z, 8);  cs.w += __shfl_xor_sync(0xffffffffu, cs.w, 8);
        cs.x += __shfl_xor_sync(0xffffffffu, cs.x, 16); cs.y += __shfl_xor_sync(0xffffffffu, cs.y, 16);
        cs.z += __shfl_xor_sync(0xffffffffu, cs.z, 16); cs.w += __shfl_xor_sync(0xffffffffu, cs.w, 16);
        if (rsub == 0 && n < N && m0 + q * 32 < M) {
          float *dstp = epi.colsum_partial + ((m0 + q * 32) >> 5) * N + n;
          const float e[4] = {cs.x, cs.y, cs.z, cs.w};
#pragma unroll
          for (int t = 0; t < 4; ++t)
            if (n + t < N) dstp[t] = e[t];
        }
      }
    }
    fence_async_smem();
    __syncwarp();
    if (lane == 0 && nb < N && m0 + q * 32 < M) {
      if (reduce) tma_reduce_add_2d(cmap, buf, (int)nb, (int)(m0 + q * 32 + row_off));
      else tma_store_2d(cmap, buf, (int)nb, (int)(m0 + q * 32 + row_off));
      bulk_commit();
    }
  }
}

// --------------------------------------------------------- persistent form of the two-CTA kernel
// One CTA pair per SM pair walks over the 256 x 256 tiles t = pair, pair + pairs, ... The ring of
// operand stages runs on across tile boundaries, so the loads of the next tile are in flight while
// the epilogue warps drain tensor memory; the MMA issuer only waits until every epilogue warp of
// both CTAs has read the accumulators into registers ("acc_empty") before it overwrites them: the
// fused epilogue and the stores of a tile run beside the products of the next one. What is saved per
// tile: the CTA launch, the tensor-memory allocation, the barrier set-up and the empty pipeline.
// The epilogue warps have 4 KB of shared memory each of their own (the stages are never free).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// Bounded wait that acquires at cluster scope (the arrivals come from both CTAs of the pair).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int code) {
  for (uint32_t it = 0; it < TC_WAIT_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  atomicCAS(&g_tc_status, 0, code);
  return false;
}

// SCHEME 0: 3xTF32, the stage holds the fp32 tile and its fp32 low part of each operand.
// SCHEME 1: the stage holds the fp32 tile (tf32 MMA hi*hi into the main accumulator) and two bf16
// tiles of half its size, bf16(x) and bf16(x - tf32(x)); the two correction products are bf16
// MMAs (K = 16 per instruction, so two per 32 k) into the second accumulator.
template <bool A_MN, bool B_MN, int SCHEME>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 1)
gemm_tc2p_kernel(const __grid_constant__ TcMaps maps, const GemmParams p, int pairs_m, int tiles_n, int group_m,
                 int ksplit, int kseq, int kseq_raw, int part_rows) {
  constexpr int BN = 256, BNH = 128, BK = 32, STAGES = 3, EPI_WARPS = 8;
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr uint32_t A_BYTES = TC_BM * BK * 4;
  constexpr uint32_t B_BYTES = BNH * BK * 4;
  constexpr uint32_t BOX_BYTES = BK * 128;
  constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  const uint32_t smem_base = (smem_u32(smem) + 1023u) & ~1023u;
  const uint32_t epi_base = smem_base + STAGES * STAGE_BYTES;
  const uint32_t bars = epi_base + EPI_WARPS * 4096u;
  __shared__ uint32_t tmem_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int num_pairs = (int)(gridDim.x >> 1), pair_id = (int)(blockIdx.x >> 1);
  // Work items: every tile once per K range (ksplit = 2 halves the reduction so that a tile count
  // that fills the last round of pairs badly is balanced; the halves are then added into a zeroed
  // C by the copy engine, and two addends give the same sum in either order). part_rows > 0: any
  // number of K ranges; range r stores its bare sums to rows [r * part_rows, ...) of the work buffer
  // behind maps.c, and splitk_finish_kernel adds the ranges in order and applies the epilogue.
  const int num_tiles = pairs_m * tiles_n * ksplit;
  const int tiles_mn = pairs_m * tiles_n;
  const int nkb_all = (int)((p.K + BK - 1) / BK);
  auto k_range = [&](int t, int &kb0, int &nkb) {
    const int part = t / tiles_mn, per = nkb_all / ksplit;
    kb0 = part * per;
    nkb = part == ksplit - 1 ? nkb_all - kb0 : per;
  };
  // Tile order: groups of group_m row-pairs; inside a group the column tiles of one row-pair band
  // follow each other, so the pairs running at the same time share a few A bands and B tiles.
  auto tile_origin = [&](int w, int &m0, int &n0) {
    const int t = w % tiles_mn;
    const int group = t / (group_m * tiles_n);
    const int gm0 = group * group_m;
    const int gh = pairs_m - gm0 < group_m ? pairs_m - gm0 : group_m;
    const int rem = t - group * (group_m * tiles_n);
    m0 = (gm0 + rem % gh) * 256 + (int)rank * 128;
    n0 = (rem / gh) * BN;
  };
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t acc_full = bars + 8u * (2 * STAGES), acc_empty = bars + 8u * (2 * STAGES + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 2 * EPI_WARPS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)(2 * BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        int m0, n0, kb0, nkb;
        tile_origin(t, m0, n0);
        k_range(t, kb0, nkb);
        const int nh0 = n0 + (int)rank * BNH;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          if (it >= STAGES && !mbar_wait(empty_bar(s), ((it / STAGES) - 1) & 1, 31)) { ok = false; break; }
          const uint32_t st = smem_base + s * STAGE_BYTES;
          if (leader) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);   // both CTAs' bytes
          const uint32_t fb = map_to_cta(full_bar(s), 0);
          const int k0 = (kb0 + kb) * BK;
          const uint32_t sb = st + 2 * A_BYTES;
          if constexpr (A_MN) {
#pragma unroll
            for (int j = 0; j < TC_BM / 32; ++j) tma_load_2d_pair(st + j * BOX_BYTES, &maps.a_hi, fb, m0 + 32 * j, k0);
          } else {
            tma_load_2d_pair(st, &maps.a_hi, fb, k0, m0);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < BNH / 32; ++j) tma_load_2d_pair(sb + j * BOX_BYTES, &maps.b_hi, fb, nh0 + 32 * j, k0);
          } else {
            tma_load_2d_pair(sb, &maps.b_hi, fb, k0, nh0);
          }
          if constexpr (SCHEME == 0) {
            if constexpr (A_MN) {
#pragma unroll
              for (int j = 0; j < TC_BM / 32; ++j)
                tma_load_2d_pair(st + A_BYTES + j * BOX_BYTES, &maps.a_lo, fb, m0 + 32 * j, k0);
            } else {
              tma_load_2d_pair(st + A_BYTES, &maps.a_lo, fb, k0, m0);
            }
            if constexpr (B_MN) {
#pragma unroll
              for (int j = 0; j < BNH / 32; ++j)
                tma_load_2d_pair(sb + B_BYTES + j * BOX_BYTES, &maps.b_lo, fb, nh0 + 32 * j, k0);
            } else {
              tma_load_2d_pair(sb + B_BYTES, &maps.b_lo, fb, k0, nh0);
            }
          } else {
            // bf16 parts: [hi16 | lo16], half a fp32 tile each
            if constexpr (A_MN) {
#pragma unroll
              for (int j = 0; j < TC_BM / 64; ++j) {
                tma_load_2d_pair(st + A_BYTES + j * 4096, &maps.a16h, fb, m0 + 64 * j, k0);
                tma_load_2d_pair(st + A_BYTES + A_BYTES / 2 + j * 4096, &maps.a16l, fb, m0 + 64 * j, k0);
              }
            } else {
              tma_load_2d_pair(st + A_BYTES, &maps.a16h, fb, k0, m0);
              tma_load_2d_pair(st + A_BYTES + A_BYTES / 2, &maps.a16l, fb, k0, m0);
            }
            if constexpr (B_MN) {
#pragma unroll
              for (int j = 0; j < BNH / 64; ++j) {
                tma_load_2d_pair(sb + B_BYTES + j * 4096, &maps.b16h, fb, nh0 + 64 * j, k0);
                tma_load_2d_pair(sb + B_BYTES + B_BYTES / 2 + j * 4096, &maps.b16l, fb, nh0 + 64 * j, k0);
              }
            } else {
              tma_load_2d_pair(sb + B_BYTES, &maps.b16h, fb, k0, nh0);
              tma_load_2d_pair(sb + B_BYTES + B_BYTES / 2, &maps.b16l, fb, k0, nh0);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) |
                             ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(256 >> 4) << 24);
      // the same with bf16 operands (format 1) for the correction products
      const uint32_t idesc16 = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                               ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                               ((uint32_t)(256 >> 4) << 24);
      (void)idesc16;
      uint32_t it = 0;
      int j = 0;
      bool ok = true;
      // kseq > 1: the reduction is cut into kseq runs; the accumulators are drained after each
      // (the first run stores, the later ones add to C), which bounds the round-toward-zero bias
      // of the accumulator adds by the length of one run. With an epilogue that is not linear in
      // the accumulator (kseq_raw) the earlier runs leave bare sums in C and the last run adds
      // them to its own before the epilogue.
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        int kb0, nkb;
        k_range(t, kb0, nkb);
        const int per_run = (nkb + kseq - 1) / kseq;
        int kb = 0;
        for (int run = 0; run < kseq && ok; ++run, ++j) {
        // the epilogue warps of both CTAs have read the previous accumulators
        if (j > 0 && !mbar_wait_cluster(acc_empty, (uint32_t)(j - 1) & 1, 32)) { ok = false; break; }
        tc_fence_after();
        const int kend = (run + 1) * per_run < nkb ? (run + 1) * per_run : nkb;
        for (int kl = 0; kb < kend; ++kb, ++kl, ++it) {
          const int s = (int)(it % STAGES);
          if (!mbar_wait(full_bar(s), (it / STAGES) & 1, 33)) { ok = false; break; }
          tc_fence_after();
          const uint32_t st = smem_base + s * STAGE_BYTES;
          const uint32_t sb = st + 2 * A_BYTES;
          const uint64_t a_hi = tile_desc<A_MN, BK>(st), b_hi = tile_desc<B_MN, BK>(sb);
          constexpr uint64_t A_STEP = A_MN ? 64 : 2, B_STEP = B_MN ? 64 : 2;
          if constexpr (SCHEME == 0) {
            const uint64_t a_lo = tile_desc<A_MN, BK>(st + A_BYTES), b_lo = tile_desc<B_MN, BK>(sb + B_BYTES);
#pragma unroll
            for (int ks = 0; ks < BK / 8; ++ks) {
              const uint64_t ah = a_hi + ks * A_STEP, al = a_lo + ks * A_STEP;
              const uint64_t bh = b_hi + ks * B_STEP, bl = b_lo + ks * B_STEP;
              const uint32_t acc = (kl | ks) ? 1u : 0u;
              // (the correction accumulator runs on over the runs of a work item)
              tc_mma_tf32_pair(tmem_base + BN, al, bh, idesc, (run | kl | ks) ? 1u : 0u);
              tc_mma_tf32_pair(tmem_base + BN, ah, bl, idesc, 1u);
              tc_mma_tf32_pair(tmem_base, ah, bh, idesc, acc);
            }
          } else {
            const uint64_t a16h = tile_desc16<A_MN>(st + A_BYTES), a16l = tile_desc16<A_MN>(st + A_BYTES + A_BYTES / 2);
            const uint64_t b16h = tile_desc16<B_MN>(sb + B_BYTES), b16l = tile_desc16<B_MN>(sb + B_BYTES + B_BYTES / 2);
            // 16 k further: 32 bytes along a K-major row, 16 k-rows (2048 bytes) of an MN-major box
            constexpr uint64_t A16_STEP = A_MN ? 128 : 2, B16_STEP = B_MN ? 128 : 2;
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks) {
              const uint32_t acc = (run | kl | ks) ? 1u : 0u;   // (runs on over the runs of a work item)
              tc_mma_bf16_pair(tmem_base + BN, a16l + ks * A16_STEP, b16h + ks * B16_STEP, idesc16, acc);
              tc_mma_bf16_pair(tmem_base + BN, a16h + ks * A16_STEP, b16l + ks * B16_STEP, idesc16, 1u);
            }
#pragma unroll
            for (int ks = 0; ks < BK / 8; ++ks)
              tc_mma_tf32_pair(tmem_base, a_hi + ks * A_STEP, b_hi + ks * B_STEP, idesc, (kl | ks) ? 1u : 0u);
          }
          tc_commit_pair(empty_bar(s));
        }
        tc_commit_pair(acc_full);   // also on the give-up path, so that the epilogue warps move on
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const uint32_t acc_empty_leader = map_to_cta(acc_empty, 0);
    int j = 0;
    bool ok = true;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
      int m0, n0;
      tile_origin(t, m0, n0);
      for (int run = 0; run < kseq; ++run, ++j) {
      if (!mbar_wait(acc_full, (uint32_t)j & 1, 34)) { ok = false; break; }
      tc_fence_after();
      constexpr int CH = BN / 64;
      static_assert(CH == 4, "the epilogue holds four chunks of 32 columns per warp");
      const bool last_run = run == kseq - 1;
      const bool raw = part_rows ? true : (kseq_raw && !last_run);
      const bool pre_add = part_rows ? false : (kseq_raw && last_run && kseq > 1);
      const bool reduce = part_rows ? run > 0 : (kseq_raw ? (run > 0 && !last_run) : (ksplit > 1 || run > 0));
      const int64_t row_off = part_rows ? (int64_t)(t / tiles_mn) * part_rows : 0;
      if (p.vec_c || part_rows) {
        // the accumulators go back to the MMA issuer as soon as they are in registers
        uint32_t v1[32], v2[32], v3[32];
        const uint32_t ebuf = epi_base + (uint32_t)(warp - 2) * 4096u;
        tc_epilogue_drain<BN>(tmem_base, q, lane, half * CH, last_run, ebuf, v1, v2, v3);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
        if (run > 0) {
          // this run is added to what the previous run of the same tile stored: that store must be complete
          if (lane == 0) bulk_wait0();
          __syncwarp();
        }
        tc_epilogue_warp_bulk(v1, v2, v3, q, lane, half * CH, m0, n0, p.M, p.N, p.C, p.ldc, p.epi, &maps.c, ebuf,
                              reduce, raw, pre_add, row_off);
      } else {
        tc_epilogue_warp<BN, false>(tmem_base, q, lane, half * CH, (half + 1) * CH, m0, n0, p.M, p.N, p.C, p.ldc,
                                    p.epi, p.vec_c, epi_base + (uint32_t)(warp - 2) * 4096u);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
      }
      }
    }
    if (lane == 0) bulk_wait0();   // the stores have left shared memory and are complete
  }
  tc_fence_before();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * BN)) : "memory");
  }
}

// Second stage of split-K: C = epilogue(sum over the splits, in order). The loads of eight splits
// are issued together; with VEC a thread takes four consecutive columns.
template <bool VEC>
__global__ void __launch_bounds__(256) splitk_finish_kernel(GemmParams p, int splits) {
  constexpr int W = VEC ? 4 : 1;
  const int64_t NW = (p.N + W - 1) / W, total = p.M * NW;
  const bool narrow = total < ((int64_t)1 << 31);
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  const int64_t slice = (p.partial_rows ? p.partial_rows : p.M) * p.ld_partial;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int64_t m = narrow ? (int64_t)((uint32_t)i / (uint32_t)NW) : i / NW;
    const int64_t n = (i - m * NW) * W;
    const float *src = p.partial + m * p.ld_partial + n;
    float v[W];
#pragma unroll
    for (int j = 0; j < W; ++j) v[j] = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 8) {
      float t[8][W];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (s0 + u < splits) {
          if (VEC) {
            const float4 q = __ldcs(reinterpret_cast<const float4 *>(src + (int64_t)(s0 + u) * slice));
            t[u][0] = q.x; t[u][W > 1 ? 1 : 0] = q.y; t[u][W > 2 ? 2 : 0] = q.z; t[u][W > 3 ? 3 : 0] = q.w;
          } else {
            t[u][0] = __ldcs(src + (int64_t)(s0 + u) * slice);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s0 + u < splits)
#pragma unroll
          for (int j = 0; j < W; ++j) v[j] += t[u][j];
    }
    float *c = p.C + m * p.ldc + n;
#pragma unroll
    for (int j = 0; j < W; ++j) v[j] = apply_epilogue(p.epi, v[j], m, n + j, c + j);
    if (VEC) *reinterpret_cast<float4 *>(c) = make_float4(v[0], v[W > 1 ? 1 : 0], v[W > 2 ? 2 : 0], v[W > 3 ? 3 : 0]);
    else c[0] = v[0];
  }
}

int launch_splitk_finish(const GemmParams &p, int splits, cudaStream_t s) {
  const bool vec = p.vec_c && p.N % 4 == 0 && p.ld_partial % 4 == 0 &&
                   (reinterpret_cast<uintptr_t>(p.partial) & 15) == 0;
  if (vec) splitk_finish_kernel<true><<<grid_for(p.M * (p.N / 4), 256), 256, 0, s>>>(p, splits);
  else splitk_finish_kernel<false><<<grid_for(p.M * p.N, 256), 256, 0, s>>>(p, splits);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

// lo = x - hi with hi = x truncated to tf32 (13 low mantissa bits cleared); exact in fp32.
// Optionally also writes hi. Rows of `cols` floats, leading dimensions ld_in / ld_out.
__global__ void __launch_bounds__(256)
tf32_split_kernel(const float *__restrict__ x, float *__restrict__ lo, float *__restrict__ hi,
                  int64_t rows, int64_t cols4, int64_t ld_in, int64_t ld_out) {
  const int64_t total = rows * cols4;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int64_t r = i / cols4, c = (i - r * cols4) * 4;
    const float4 v = __ldg(reinterpret_cast<const float4 *>(x + r * ld_in + c));
    float4 h, l;
    h.x = __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u); l.x = v.x - h.x;
    h.y = __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u); l.y = v.y - h.y;
    h.z = __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u); l.z = v.z - h.z;
    h.w = __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u); l.w = v.w - h.w;
    *reinterpret_cast<float4 *>(lo + r * ld_out + c) = l;
    if (hi) *reinterpret_cast<float4 *>(hi + r * ld_out + c) = h;
  }
}

int launch_tf32_split(const float *x, float *lo, int64_t rows, int64_t cols, int64_t ld_in, int64_t ld_out,
                      cudaStream_t s) {
  tf32_split_kernel<<<grid_for(rows * (cols / 4), 256), 256, 0, s>>>(x, lo, nullptr, rows, cols / 4, ld_in, ld_out);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

// hi16 = bf16(x) and lo16 = bf16(x - tf32(x)), round to nearest; the operand parts of the
// bf16-compensated scheme. Rows of `cols` floats, leading dimensions ld_in (floats) / ld_out (bf16).
__global__ void __launch_bounds__(256)
bf16_split_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo,
                  int64_t rows, int64_t cols4, int64_t ld_in, int64_t ld_out) {
  const int64_t total = rows * cols4;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int64_t r = i / cols4, c = (i - r * cols4) * 4;
    const float4 v = __ldg(reinterpret_cast<const float4 *>(x + r * ld_in + c));
    const float l0 = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
    const float l1 = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
    const float l2 = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
    const float l3 = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
    __nv_bfloat162 h01 = __floats2bfloat162_rn(v.x, v.y), h23 = __floats2bfloat162_rn(v.z, v.w);
    __nv_bfloat162 l01 = __floats2bfloat162_rn(l0, l1), l23 = __floats2bfloat162_rn(l2, l3);
    uint2 hv, lv;
    hv.x = *reinterpret_cast<uint32_t *>(&h01); hv.y = *reinterpret_cast<uint32_t *>(&h23);
    lv.x = *reinterpret_cast<uint32_t *>(&l01); lv.y = *reinterpret_cast<uint32_t *>(&l23);
    *reinterpret_cast<uint2 *>(hi + r * ld_out + c) = hv;
    *reinterpret_cast<uint2 *>(lo + r * ld_out + c) = lv;
  }
}

int launch_bf16_split(const float *x, void *hi16, void *lo16, int64_t rows, int64_t cols, int64_t ld_in,
                      int64_t ld_out, cudaStream_t s) {
  bf16_split_kernel<<<grid_for(rows * (cols / 4), 256), 256, 0, s>>>(
      x, static_cast<__nv_bfloat16 *>(hi16), static_cast<__nv_bfloat16 *>(lo16), rows, cols / 4, ld_in, ld_out);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

int tc_default_scheme() {
  static const int scheme = []() {
    const char *e = getenv("ENDIA_B200_TC_SCHEME");
    return (e && (e[0] == '3' || e[0] == '0')) ? 0 : 1;
  }();
  return scheme;
}

// ---------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    else
      cudaGetLastError();
  }
  return fn;
}

// Tensor map over a row-major [outer, inner] float array with leading dimension ld; the box is
// [box_outer, box_inner] floats; out-of-range elements read as zero. MN-major tiles (32 floats
// wide) use the 128-byte swizzle in 32-byte units, K-major tiles the swizzle as wide as a row.
static int make_map(CUtensorMap *map, const float *base, int64_t inner, int64_t outer, int64_t ld,
                    int box_inner, int box_outer, bool mn_major) {
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims,
                           strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                    : (box_inner == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B),
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("gemm: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return ENDIA_B200_ECUDA;
  }
  return ENDIA_B200_OK;
}

// Tensor map over a row-major [outer, inner] bf16 array with leading dimension ld (elements).
// K-major tiles: box [box_outer rows][32 k] with the 64-byte swizzle; MN-major tiles: box
// [32 k][64 rows] with the 128-byte swizzle.
static int make_map16(CUtensorMap *map, const void *base, int64_t inner, int64_t outer, int64_t ld,
                      int box_inner, int box_outer, bool mn_major) {
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           mn_major ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("gemm: cuTensorMapEncodeTiled (bf16) failed with code %d", (int)r);
    return ENDIA_B200_ECUDA;
  }
  return ENDIA_B200_OK;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

bool tc_gemm_supported(const GemmParams &p, int trans_a, int trans_b, int64_t batch, bool explicit_request) {
  (void)trans_a; (void)trans_b;
  if (batch != 1) return false;
  // the fused column sum lives in the epilogue of the two-CTA kernel only
  if (p.epi.colsum_partial && (p.N < 256 || !p.vec_c)) return false;
  // The tensor-core accumulator rounds toward zero on every add, a bias that grows linearly
  // with K (measured: -1.7e-5 of the result at K = 8192, -6.7e-5 at K = 32768). Longer
  // reductions stay on the FFMA kernel unless the caller asks for this one by name.
  // The two-CTA kernel is exempt where it can cut the reduction into short runs (see
  // launch_gemm_tc): a linear epilogue, or any epilogue with beta == 0.
  const bool linear = !p.epi.bias && !p.epi.act && !p.epi.dact && p.epi.beta == 0.f && !p.epi.colsum_partial;
  const bool runs_ok = p.N >= 256 && p.vec_c && (linear || p.epi.beta == 0.f);
  if (p.K > 8192 && !explicit_request && !runs_ok) return false;
  if (!encode_fn()) return false;
  if (p.M < 128 || p.N < 128 || p.K < 32) return false;      // small products stay on the FFMA kernel
  if (p.M > (int64_t)1 << 30 || p.N > (int64_t)1 << 30 || p.K > (int64_t)1 << 30) return false;
  if (!aligned16(p.A) || !aligned16(p.B) || p.lda % 4 || p.ldb % 4) return false;
  return true;
}

template <int BN, int BK, int STAGES>
static int launch_variant(const TcMaps &maps, const GemmParams &p, int trans_a, int trans_b,
                          cudaStream_t s, int splits = 1) {
  constexpr size_t SMEM = (size_t)STAGES * (2 * TC_BM * BK * 4 + 2 * BN * BK * 4) + 1024 + 256;
  const int tiles_m = (int)ceil_div(p.M, TC_BM), tiles_n = (int)ceil_div(p.N, BN);
  const dim3 grid((unsigned)(tiles_m * tiles_n), (unsigned)splits);
#define EB_TC_LAUNCH(AM, BM_)                                                                     \
  do {                                                                                            \
    auto kern = gemm_tc_kernel<BN, BK, STAGES, AM, BM_>;                                              \
    static bool attr = false;                                                                     \
    if (!attr) {                                                                                  \
      EB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM)); \
      attr = true;                                                                                \
    }                                                                                             \
    kern<<<grid, 320, SMEM, s>>>(maps, p, tiles_m);                                               \
  } while (0)
  if (trans_a && !trans_b) EB_TC_LAUNCH(true, true);
  else if (trans_a && trans_b) EB_TC_LAUNCH(true, false);
  else if (!trans_a && !trans_b) EB_TC_LAUNCH(false, true);
  else EB_TC_LAUNCH(false, false);
#undef EB_TC_LAUNCH
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

static bool pair_mode() {
  static const bool on = []() { const char *e = getenv("ENDIA_B200_TC_PAIR"); return !(e && atoi(e) == 0); }();
  return on;
}

// K ranges as work items of the two-CTA kernel when a product has few tiles (ENDIA_B200_TC_PAIR_SPLIT=0: off)
static bool pair_split_mode() {
  static const bool on = []() { const char *e = getenv("ENDIA_B200_TC_PAIR_SPLIT"); return !(e && atoi(e) == 0); }();
  return on;
}

// CTA pairs the persistent kernel runs with (SM pairs minus the reserve for concurrent kernels).
static int pair_capacity() {
  static const int cap = []() {
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const char *rs = getenv("ENDIA_B200_TC_RESERVE_SMS");
    const int c = sms / 2 - (rs ? atoi(rs) / 2 : 0);
    return c >= 8 ? c : 8;
  }();
  return cap;
}

static bool ksplit_mode() {
  static const bool on = []() { const char *e = getenv("ENDIA_B200_TC_KSPLIT"); return !(e && atoi(e) == 0); }();
  return on;
}

// Persistent two-CTA kernel: as many CTA pairs as can be resident, each walking over its tiles.
template <int SCHEME>
static int launch_pair_persistent(const TcMaps &maps, const GemmParams &p, int trans_a, int trans_b,
                                  cudaStream_t s, int ksplit_max, int run_k, int kseq_raw, int part_splits) {
  // part_splits >= 2: that many K ranges per tile, each with its slice of the work buffer behind
  // maps.c (pairs_m * 256 rows per slice)
  constexpr size_t SMEM = (size_t)3 * (2 * TC_BM * 32 * 4 + 2 * 128 * 32 * 4) + 8 * 4096 + 1024 + 256;
  const int pairs_m = (int)ceil_div(p.M, 256), tiles_n = (int)ceil_div(p.N, 256);
  static const int group_env = []() { const char *e = getenv("ENDIA_B200_TC_GROUP_M"); return e ? atoi(e) : TC_GROUP_M; }();
  const int group_m = group_env > 0 ? group_env : pairs_m;
#define EB_TC2P_LAUNCH(AM, BM_)                                                                   \
  do {                                                                                            \
    auto kern = gemm_tc2p_kernel<AM, BM_, SCHEME>;                                                \
    static int max_pairs = 0;                                                                     \
    if (!max_pairs) {                                                                             \
      EB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM)); \
      cudaLaunchConfig_t cfg = {};                                                                \
      cfg.gridDim = dim3(2);                                                                      \
      cfg.blockDim = dim3(320);                                                                   \
      cfg.dynamicSmemBytes = SMEM;                                                                \
      cudaLaunchAttribute at;                                                                     \
      at.id = cudaLaunchAttributeClusterDimension;                                                \
      at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;                  \
      cfg.attrs = &at;                                                                            \
      cfg.numAttrs = 1;                                                                           \
      int nc = 0;                                                                                 \
      if (cudaOccupancyMaxActiveClusters(&nc, kern, &cfg) != cudaSuccess || nc <= 0) {            \
        cudaGetLastError();                                                                       \
        int dev = 0, sms = 0;                                                                     \
        cudaGetDevice(&dev);                                                                      \
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);                        \
        nc = sms / 2;                                                                             \
      }                                                                                           \
      /* SMs left free for kernels that run beside the GEMMs (a collective on another stream): a \
         pair that cannot become resident would otherwise start its share of the tiles late */    \
      const char *rs = getenv("ENDIA_B200_TC_RESERVE_SMS");                                       \
      const int reserve = rs ? atoi(rs) / 2 : 0;                                                  \
      max_pairs = nc - reserve >= 8 ? nc - reserve : (nc >= 8 ? 8 : nc);                          \
    }                                                                                             \
    const int tiles = pairs_m * tiles_n;                                                          \
    int ksplit = 1;                                                                               \
    if (part_splits >= 2) {                                                                       \
      ksplit = part_splits;                                                                       \
    } else if (ksplit_max >= 2 && tiles > max_pairs) {                                                   \
      /* rounds of pairs with and without halving K, in units of half tiles */                    \
      const int r1 = 2 * ((tiles + max_pairs - 1) / max_pairs);                                   \
      const int r2 = (2 * tiles + max_pairs - 1) / max_pairs;                                     \
      if (r2 * 100 <= r1 * 95) ksplit = 2;                                                        \
    }                                                                                             \
    if (ksplit > 1 && part_splits < 2) {                                                          \
      if (p.ldc == p.N) EB_CUDA(cudaMemsetAsync(p.C, 0, sizeof(float) * p.M * p.N, s));           \
      else EB_CUDA(cudaMemset2DAsync(p.C, sizeof(float) * p.ldc, 0, sizeof(float) * p.N, p.M, s)); \
    }                                                                                             \
    const int items = tiles * ksplit;                                                             \
    const int pairs = items < max_pairs ? items : max_pairs;                                      \
    /* runs of at most run_k along K per work item (run_k = 0: one run) */                        \
    const int kseq = run_k > 0 ? (int)ceil_div(ceil_div(p.K, ksplit), run_k) : 1;                 \
    kern<<<dim3((unsigned)(2 * pairs)), 320, SMEM, s>>>(maps, p, pairs_m, tiles_n, group_m, ksplit,  \
                                                        kseq < 1 ? 1 : kseq, kseq > 1 ? kseq_raw : 0,   \
                                                        part_splits >= 2 ? pairs_m * 256 : 0);        \
  } while (0)
  if (trans_a && !trans_b) EB_TC2P_LAUNCH(true, true);
  else if (trans_a && trans_b) EB_TC2P_LAUNCH(true, false);
  else if (!trans_a && !trans_b) EB_TC2P_LAUNCH(false, true);
  else EB_TC2P_LAUNCH(false, false);
#undef EB_TC2P_LAUNCH
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

int launch_gemm_tc(const GemmParams &p_in, int trans_a, int trans_b, cudaStream_t s, bool *c16_written) {
  GemmParams p = p_in;
  if (c16_written) *c16_written = false;
  // Operand geometry in memory: A is [M, K] (K-major) or [K, M] (MN-major); B is [K, N] (MN-major,
  // the row-major weight of `x @ W`) or [N, K] (K-major).
  const int64_t a_rows = trans_a ? p.K : p.M, a_cols = trans_a ? p.M : p.K;
  const int64_t b_rows = trans_b ? p.N : p.K, b_cols = trans_b ? p.K : p.N;
  int bn = p.N >= 256 ? 256 : 128;
  // Few output tiles and a long reduction: split K over CTAs (128 x 128 tiles) so that the machine
  // is filled; the partial sums go through a work buffer and are added in a fixed order.
  // N >= 256: the two-CTA kernel takes K ranges as extra work items (part_splits), each with its
  // own slice of a work buffer; N < 256: the one-CTA kernel, 128 x 128 tiles (splits).
  int splits = 1, part_splits = 1;
  int scheme = p.scheme;
  if (bn == 256 && !p.epi.colsum_partial && p.K >= 2048 && pair_split_mode()) {
    const int64_t tiles = ceil_div(p.M, 256) * ceil_div(p.N, 256);
    const int64_t cap = pair_capacity();
    if (2 * tiles <= cap) {
      int64_t sp = cap / tiles;
      if (sp > p.K / 512) sp = p.K / 512;
      if (sp > 16) sp = 16;
      if (sp >= 2) part_splits = (int)sp;
    }
  } else if (bn == 128 && (scheme == 0 || !p.scheme_forced) && !p.epi.colsum_partial && p.K <= 8192) {
    const int64_t tiles = ceil_div(p.M, 128) * ceil_div(p.N, 128);
    const int64_t nkb32 = ceil_div(p.K, 32);
    if (tiles < 100 && nkb32 >= 16) {
      int64_t sp = 148 / tiles;
      if (sp > nkb32 / 8) sp = nkb32 / 8;
      if (sp > 16) sp = 16;
      if (sp >= 2) { splits = (int)sp; scheme = 0; }
    }
  }
  // k-block depth of the one-CTA kernel: 32 floats per stage, or 16 with a deeper ring.
  static const int bk = []() {
    const char *e = getenv("ENDIA_B200_TC_BK");
    return (e && atoi(e) == 16) ? 16 : 32;
  }();
  const bool pair = bn == 256 && ((bk == 32 && pair_mode()) || scheme == 1 || p.epi.colsum_partial);
  const bool bf16c = pair && scheme == 1;
  TcMaps maps;
  int st;
  // K-major operand: box [rows of the tile][k]; MN-major operand: box [k][32 rows].
  const int kbox = pair ? 32 : bk;
  const int a_bi = trans_a ? 32 : kbox, a_bo = trans_a ? kbox : TC_BM;
  const int b_bi = trans_b ? kbox : 32, b_bo = trans_b ? (pair ? 128 : bn) : kbox;
  if ((st = make_map(&maps.a_hi, p.A, a_cols, a_rows, p.lda, a_bi, a_bo, trans_a != 0))) return st;
  if ((st = make_map(&maps.b_hi, p.B, b_cols, b_rows, p.ldb, b_bi, b_bo, trans_b == 0))) return st;
  maps.a_lo = maps.a16h = maps.a16l = maps.a_hi;
  maps.b_lo = maps.b16h = maps.b16l = maps.b_hi;

  // Operand parts: taken from the caller when provided (laid out like the operand's storage), else
  // computed into stream-ordered work buffers.
  // (stream-ordered work buffers, released on every way out of this function)
  struct WorkBuffers {
    cudaStream_t s;
    void *a = nullptr, *b = nullptr, *partial = nullptr;
    ~WorkBuffers() {
      if (a) cudaFreeAsync(a, s);
      if (b) cudaFreeAsync(b, s);
      if (partial) cudaFreeAsync(partial, s);
    }
  } work{s};
  void *&a_buf = work.a, *&b_buf = work.b;
  if (bf16c) {
    // bf16(x) and bf16(x - tf32(x)), each [rows][ld16] bf16
    const int64_t a_ld16 = (a_cols + 7) / 8 * 8, b_ld16 = (b_cols + 7) / 8 * 8;
    const char *a16 = static_cast<const char *>(p.a16), *b16 = static_cast<const char *>(p.b16);
    int64_t a_ld = p.lda, b_ld = p.ldb;
    if (!a16 || p.lda % 8 || !aligned16(a16)) {
      EB_CUDA(cudaMallocAsync(&a_buf, (size_t)4 * a_rows * a_ld16, s));
      if ((st = launch_bf16_split(p.A, a_buf, static_cast<char *>(a_buf) + 2 * a_rows * a_ld16, a_rows,
                                  (a_cols + 3) / 4 * 4 <= a_ld16 ? (a_cols + 3) / 4 * 4 : a_cols, p.lda, a_ld16, s)))
        return st;
      a16 = static_cast<const char *>(a_buf); a_ld = a_ld16;
    }
    if (!b16 || p.ldb % 8 || !aligned16(b16)) {
      EB_CUDA(cudaMallocAsync(&b_buf, (size_t)4 * b_rows * b_ld16, s));
      if ((st = launch_bf16_split(p.B, b_buf, static_cast<char *>(b_buf) + 2 * b_rows * b_ld16, b_rows,
                                  (b_cols + 3) / 4 * 4 <= b_ld16 ? (b_cols + 3) / 4 * 4 : b_cols, p.ldb, b_ld16, s)))
        return st;
      b16 = static_cast<const char *>(b_buf); b_ld = b_ld16;
    }
    // K-major: box [tile rows][32 k]; MN-major: box [32 k][64 rows]
    const int a16_bi = trans_a ? 64 : 32, a16_bo = trans_a ? 32 : TC_BM;
    const int b16_bi = trans_b ? 32 : 64, b16_bo = trans_b ? 128 : 32;
    if ((st = make_map16(&maps.a16h, a16, a_cols, a_rows, a_ld, a16_bi, a16_bo, trans_a != 0))) return st;
    if ((st = make_map16(&maps.a16l, a16 + 2 * a_rows * a_ld, a_cols, a_rows, a_ld, a16_bi, a16_bo, trans_a != 0))) return st;
    if ((st = make_map16(&maps.b16h, b16, b_cols, b_rows, b_ld, b16_bi, b16_bo, trans_b == 0))) return st;
    if ((st = make_map16(&maps.b16l, b16 + 2 * b_rows * b_ld, b_cols, b_rows, b_ld, b16_bi, b16_bo, trans_b == 0))) return st;
  } else {
    const int64_t a_ld4 = (a_cols + 3) / 4 * 4, b_ld4 = (b_cols + 3) / 4 * 4;
    const float *a_lo = p.a_lo, *b_lo = p.b_lo;
    int64_t a_lo_ld = p.lda, b_lo_ld = p.ldb;
    if (!a_lo) {
      EB_CUDA(cudaMallocAsync(&a_buf, sizeof(float) * a_rows * a_ld4, s));
      if ((st = launch_tf32_split(p.A, static_cast<float *>(a_buf), a_rows, a_ld4, p.lda, a_ld4, s))) return st;
      a_lo = static_cast<const float *>(a_buf); a_lo_ld = a_ld4;
    }
    if (!b_lo) {
      EB_CUDA(cudaMallocAsync(&b_buf, sizeof(float) * b_rows * b_ld4, s));
      if ((st = launch_tf32_split(p.B, static_cast<float *>(b_buf), b_rows, b_ld4, p.ldb, b_ld4, s))) return st;
      b_lo = static_cast<const float *>(b_buf); b_lo_ld = b_ld4;
    }
    if ((st = make_map(&maps.a_lo, a_lo, a_cols, a_rows, a_lo_ld, a_bi, a_bo, trans_a != 0))) return st;
    if ((st = make_map(&maps.b_lo, b_lo, b_cols, b_rows, b_lo_ld, b_bi, b_bo, trans_b == 0))) return st;
  }
  GemmParams q = p;
  if (splits > 1) {
    q.ld_partial = (p.N + 3) / 4 * 4;
    EB_CUDA(cudaMallocAsync(&work.partial, sizeof(float) * (size_t)splits * p.M * q.ld_partial, s));
    q.partial = static_cast<float *>(work.partial);
  }
  if (!pair) part_splits = 1;
  if (part_splits >= 2) {
    // work buffer [part_splits][rows of whole tiles][N]: the kernel stores bare sums, the finishing
    // kernel adds the slices in order and applies the epilogue
    q.ld_partial = (p.N + 3) / 4 * 4;
    q.partial_rows = ceil_div(p.M, 256) * 256;
    EB_CUDA(cudaMallocAsync(&work.partial, sizeof(float) * (size_t)part_splits * q.partial_rows * q.ld_partial, s));
    q.partial = static_cast<float *>(work.partial);
    if ((st = make_map(&maps.c, q.partial, p.N, (int64_t)part_splits * q.partial_rows, q.ld_partial, 32, 32, false)))
      return st;
  } else if (pair && p.vec_c) {
    // output map: [M][N] floats with leading dimension ldc, boxes of 32 rows x 32 floats
    if ((st = make_map(&maps.c, p.C, p.N, p.M, p.ldc, 32, 32, false))) return st;
  } else {
    maps.c = maps.a_hi;
  }
  // Halving K needs the bulk-store epilogue, a product that is linear in the accumulator and a
  // reduction long enough for the second pass over C to be cheap.
  // The operand parts of C are written by the bulk-store epilogue of the two-CTA kernel only (from
  // the final values, so the epilogue then counts as not linear); elsewhere the caller splits C.
  if (!(pair && p.vec_c) || part_splits >= 2) p.epi.c16 = nullptr;
  if (c16_written) *c16_written = p.epi.c16 != nullptr;
  const bool linear_epi = !p.epi.bias && !p.epi.act && !p.epi.dact && p.epi.beta == 0.f && !p.epi.colsum_partial &&
                          !p.epi.c16;
  const int ksplit_max = (p.vec_c && linear_epi && p.K >= 4096 && ksplit_mode()) ? 2 : 1;
  // The tensor-core accumulator rounds toward zero, a bias that grows with the number of adds
  // into one accumulator: the reduction runs as ceil(K / run_k) runs whose sums are added in
  // order in fp32 (round to nearest). An epilogue that is linear in the accumulator is applied
  // per run; any other (bias, activation, mask, column sums) needs beta == 0, because the runs
  // before the last keep their bare sums in C.
  static const int run_k_env = []() { const char *e = getenv("ENDIA_B200_TC_RUN_K"); return e ? atoi(e) : 2048; }();
  const bool runs_ok = pair && (part_splits >= 2 || (p.vec_c && (linear_epi || p.epi.beta == 0.f)));
  const int run_k = runs_ok ? (run_k_env > 0 ? (run_k_env + 31) / 32 * 32 : 0) : 0;
  const int kseq_raw = linear_epi ? 0 : 1;
  if (bf16c) st = launch_pair_persistent<1>(maps, p, trans_a, trans_b, s, ksplit_max, run_k, kseq_raw, part_splits);
  else if (pair) st = launch_pair_persistent<0>(maps, p, trans_a, trans_b, s, ksplit_max, run_k, kseq_raw, part_splits);
  else if (bn == 256 && bk == 16) st = launch_variant<256, 16, 4>(maps, p, trans_a, trans_b, s);
  else if (bn == 256) st = launch_variant<256, 32, 2>(maps, p, trans_a, trans_b, s);
  else if (bk == 16) st = launch_variant<128, 16, 6>(maps, q, trans_a, trans_b, s, splits);
  else st = launch_variant<128, 32, 3>(maps, q, trans_a, trans_b, s, splits);
  if (splits > 1 && st == ENDIA_B200_OK) st = launch_splitk_finish(q, splits, s);
  if (part_splits >= 2 && st == ENDIA_B200_OK) st = launch_splitk_finish(q, part_splits, s);
  return st;
}

int tc_status_and_clear(cudaStream_t s) {
  int h = 0;
  if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&h, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
  if (h) {
    int z = 0;
    cudaMemcpyToSymbol(g_tc_status, &z, sizeof(int));
  }
  return h;
}

}  // namespace eb


extern "C" int endia_b200_has_tcgen05(void) { return eb::encode_fn() != nullptr ? 1 : 0; }

extern "C" int endia_b200_selftest_wait_timeout(int32_t polls, void *stream) {
  int st = eb::require_device();
  if (st) return st;
  EB_REQUIRE(polls >= 1 && polls <= (1 << 20), ENDIA_B200_EINVAL, "selftest_wait_timeout: polls must be in [1, 2^20]");
  eb::wait_selftest_kernel<<<1, 32, 0, eb::as_stream(stream)>>>((uint32_t)polls);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

extern "C" int endia_b200_device_status(void *stream) {
  int st = eb::require_device();
  if (st) return st;
  int code = eb::tc_status_and_clear(eb::as_stream(stream));
  if (code < 0) {
    eb::set_error("device_status: synchronising the stream failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ENDIA_B200_ECUDA;
  }
  if (code > 0) {
    eb::set_error("a bounded device-side wait gave up (tcgen05 GEMM, wait code %d)", code);
    return ENDIA_B200_ETIMEOUT;
  }
  return ENDIA_B200_OK;
}
