// What the two tcgen05 prefill attention kernels share: barriers with bounded waits, TMA loads,
// matrix descriptors, the tcgen05 instructions, and the tensor maps of queries, cache pages and
// gate. Included inside each kernel's file, after HEAD_DIM and GROUP are known.
#pragma once
#include <cuda.h>

#include "common.cuh"

#define OMNIA_ERR_TIMEOUT 8

namespace {

typedef __nv_bfloat16 bf16;

constexpr uint32_t WAIT_LIMIT = 1u << 20;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.f;  // log2 of how far a row's maximum may outgrow its exponent offset

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"  // sleeps up to the hint (ns)
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(2000u)
      : "memory");
  return ok != 0;
}
// Bounded wait; false when the block is giving up (its own limit, or another role's).
// 1 / (1 + e^-x) = (1 + tanh(x / 2)) / 2 for a pair of bfloat16 gate values, from the hardware's
// packed tanh: one trip to the special-function unit per PAIR, the result rounded to bfloat16 (the
// reference, too, rounds the gate's sigmoid to the activations' type before it multiplies:
// src/mlx_omnia/engine/core/attention.py:673-681). That unit is what the epilogue waits for: the
// softmax of the block next door keeps it three quarters busy, and an operation that should take a
// warp 8 cycles takes 40 to 80 there. Of a block's 5.6 us of epilogue the sigmoids are 2.9 and the
// gate's reads from shared memory 1.3 (an exponential and a reciprocal per value: 6.3 us in all).
__device__ __forceinline__ float2 sigmoid_pair(uint32_t gates) {
  const __nv_bfloat162 half = __floats2bfloat162_rn(0.5f, 0.5f);
  const __nv_bfloat162 x = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&gates), half);
  uint32_t t;
  asm("tanh.approx.bf16x2 %0, %1;" : "=r"(t) : "r"(*reinterpret_cast<const uint32_t*>(&x)));
  return __bfloat1622float2(__hfma2(*reinterpret_cast<const __nv_bfloat162*>(&t), half, half));
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (omnia_mbar_test(bar, parity)) return true;
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try(bar, parity)) return true;
    if ((i & 63) == 63 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Matrix descriptors of 128-byte-swizzled tiles (rows of 128 bytes, 8-row groups 1024 bytes apart).
// K-major: the contraction index runs along the 128-byte row. MN-major: the other index does, and
// a second 64-wide half of that index lies `leading` bytes away.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t leading) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((leading >> 4) & 0x3FFF) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16: float32 accumulator, bfloat16 operands, A K-major, B K-major or MN-major.
__host__ __device__ constexpr uint32_t idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t instr, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(instr), "r"(accumulate)
      : "memory");
}
// The same with the A operand in tensor memory (rows on the lanes, two 16-bit elements per column).
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t instr, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(instr), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load32(uint32_t addr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(addr));
}
__device__ __forceinline__ void tmem_load8(uint32_t addr, uint32_t* v) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(addr));
}
__device__ __forceinline__ void tmem_store32(uint32_t addr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void tmem_store8(uint32_t addr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

#ifdef ATTN_TIMING
// Debug build only: nanosecond stamps of block (0, 0), read back with omnia_attention_timing.
__device__ unsigned long long g_timing[8192];
__device__ __forceinline__ void stamp(int slot) {
  if (blockIdx.x == 0 && slot < 8192) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_timing[slot] = t;
  }
}
#define STAMP(role, j, what) stamp(((j) * 4 + (what)) * 4 + (role))
#else
#define STAMP(role, j, what)
#endif


// ---- host side: the tensor maps ----------------------------------------------------------------

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* symbol = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(symbol);
  }
  return fn;
}


// q: [tokens, nq, head_dim], a box is `tokens_per_block` tokens x `group` heads x 64 dims; pages:
// [num_pages, 2, nkv, page_size, head_dim] as rows of head_dim, a box is 16 keys x 64 dims; the gate's
// rows as q's are, in the matrix they are columns of, if TMA can address them (*gate_tma says so).
inline int attention_maps(CUtensorMap* map_q, CUtensorMap* map_kv, CUtensorMap* map_gate, int* gate_tma,
                          const void* q, int tokens, const void* pages, const void* gate, int gate_stride,
                          int num_pages, int nq, int nkv, int page_size, int head_dim, int group, int tokens_per_block) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return (int)cudaErrorNotSupported;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)nq, (cuuint64_t)tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)nq * head_dim * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)tokens_per_block};
    const cuuint32_t elem[3] = {1, 1, 1};
    if (encode(map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return (int)cudaErrorInvalidValue;
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)num_pages * 2 * nkv * page_size};
    const cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
    const cuuint32_t box[2] = {64, 16};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return (int)cudaErrorInvalidValue;
  }
  *map_gate = *map_q;
  *gate_tma = gate != nullptr && ((uintptr_t)gate & 15) == 0 && gate_stride % 8 == 0 && gate_stride >= nq * head_dim;
  if (*gate_tma) {
    const cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)nq, (cuuint64_t)tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)gate_stride * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)tokens_per_block};
    const cuuint32_t elem[3] = {1, 1, 1};
    if (encode(map_gate, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(gate), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return (int)cudaErrorInvalidValue;
  }
  return 0;
}

}  // namespace
