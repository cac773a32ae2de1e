// out[m, n] = sum_k a[m, k] * w[n, k] for up to 64 rows m (decode steps): the weight
// matrix is streamed from HBM exactly once, straight into tensor-core fragments.
//
// A warp owns 16 (or 32) weight rows and one slice of k. The m16n8k16 MMA takes the weight
// rows as its 16-row operand and 8 activation rows as its 8-column operand (up to eight such
// tiles of activations per pass over the weights). A dot
// product does not care about the order of k, so every thread loads 16 contiguous bytes
// (8 values of k) of its weight row and the same 8 values of k of its activation row, and
// feeds them to two MMAs; no shared memory and no shuffles are needed to form fragments.
// The eight warps of a block take eight slices of k and add their partial sums through
// shared memory in a fixed order, so results do not depend on timing.
//
// Epilogues: plain store; SwiGLU (the block computes row n of the gate half and row n of
// the up half and stores silu(gate) * up); soft cap (float32 logits = cap * tanh(z * mult / cap)).
// bfloat16 operands, float32 accumulation. k must be a multiple of 8.
#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_SOFTCAP = 2 };

__device__ __forceinline__ uint4 load_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16(float* c, unsigned a0, unsigned a1, unsigned a2,
                                         unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: activation tiles of 8 rows (1, 2, 4 or 8). RG: weight row groups of 16 per warp (1 or 2).
// With EPI_SWIGLU, RG is 2 and the second group lies `pair_offset` rows after the first.
// UNROLL: k-blocks whose loads are issued together (fewer when many activation tiles need registers).
// WARPS: slices of k per block (8, or 16 for matrices with so few rows that the grid is one wave).
template <int NT, int RG, int EPI, int WARPS, int UNROLL = (NT <= 2 ? 4 : 2)>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, void* __restrict__ out,
                   int m, int n, int k, int pair_offset, float multiplier, float cap) {
  extern __shared__ float partial_raw[];
  float (*partial)[RG * 16][NT * 8 + 1] = reinterpret_cast<float (*)[RG * 16][NT * 8 + 1]>(partial_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rows_per_block = EPI == EPI_SWIGLU ? 16 : RG * 16;
  const int n0 = blockIdx.x * rows_per_block;

  // Weight rows of this thread: group r covers rows base_r + g and base_r + g + 8.
  const bf16* wrow[RG][2];
  bool wlive[RG][2];
#pragma unroll
  for (int r = 0; r < RG; ++r)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = n0 + (EPI == EPI_SWIGLU ? r * pair_offset : r * 16) + g + 8 * h;
      const int limit = EPI == EPI_SWIGLU ? (r + 1) * pair_offset : n;
      wlive[r][h] = row < limit && row < n;
      wrow[r][h] = w + (size_t)(wlive[r][h] ? row : 0) * k;
    }
  const bf16* arow[NT];
  bool alive[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    alive[j] = 8 * j + g < m;
    arow[j] = a + (size_t)(alive[j] ? 8 * j + g : 0) * k;
  }

  float acc[RG][NT][4];
#pragma unroll
  for (int r = 0; r < RG; ++r)
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[r][j][0] = acc[r][j][1] = acc[r][j][2] = acc[r][j][3] = 0.f;

  const int blocks = (k + 31) / 32;
  const int per_warp = (blocks + WARPS - 1) / WARPS;
  const int b_begin = warp * per_warp, b_end = min(blocks, b_begin + per_warp);
  const uint4 zero = make_uint4(0, 0, 0, 0);
  // The weights do not depend on the kernel before this one: pull this warp's slice of them into
  // L2 while that kernel is still finishing, then wait for the activations it produces.
  {
    const int slice_begin = b_begin * 64, slice_end = min(b_end * 64, k * 2);  // bytes within a row
#pragma unroll
    for (int r = 0; r < RG; ++r)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        if (wlive[r][h])
          for (int off = slice_begin + t * 128; off < slice_end; off += 512)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(wrow[r][h]) + off));
  }
  pdl_wait();
  for (int b0 = b_begin; b0 < b_end; b0 += UNROLL) {
    uint4 wv[UNROLL][RG][2], av[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kk = (b0 + u) * 32 + 8 * t;
      const bool live = b0 + u < b_end && kk < k;
#pragma unroll
      for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int h = 0; h < 2; ++h) wv[u][r][h] = live && wlive[r][h] ? load_stream(wrow[r][h] + kk) : zero;
#pragma unroll
      for (int j = 0; j < NT; ++j)
        av[u][j] = live && alive[j] ? __ldcg(reinterpret_cast<const uint4*>(arow[j] + kk)) : zero;
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          mma_bf16(acc[r][j], wv[u][r][0].x, wv[u][r][1].x, wv[u][r][0].y, wv[u][r][1].y, av[u][j].x, av[u][j].y);
          mma_bf16(acc[r][j], wv[u][r][0].z, wv[u][r][1].z, wv[u][r][0].w, wv[u][r][1].w, av[u][j].z, av[u][j].w);
        }
  }
  // The weights are read: the next kernel may start its own preamble while the sums are reduced.
  pdl_launch_dependents();
  // Partial sums: C fragment (row g / g + 8 of the group, activation rows 2t, 2t + 1).
#pragma unroll
  for (int r = 0; r < RG; ++r)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      partial[warp][r * 16 + g][j * 8 + 2 * t] = acc[r][j][0];
      partial[warp][r * 16 + g][j * 8 + 2 * t + 1] = acc[r][j][1];
      partial[warp][r * 16 + g + 8][j * 8 + 2 * t] = acc[r][j][2];
      partial[warp][r * 16 + g + 8][j * 8 + 2 * t + 1] = acc[r][j][3];
    }
  __syncthreads();
  const int out_rows = EPI == EPI_SWIGLU ? 16 : RG * 16;
  for (int idx = threadIdx.x; idx < out_rows * NT * 8; idx += WARPS * 32) {
    const int token = idx / out_rows, row = idx % out_rows;
    if (token >= m) continue;
    float v = 0.f;
#pragma unroll
    for (int s = 0; s < WARPS; ++s) v += partial[s][row][token];
    if (EPI == EPI_SWIGLU) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < WARPS; ++s) u += partial[s][16 + row][token];
      const int col = n0 + row;
      if (col >= pair_offset) continue;
      // The two halves are rounded to bfloat16 first, as a separate product would round them.
      const float gate = __bfloat162float(__float2bfloat16_rn(v)), up = __bfloat162float(__float2bfloat16_rn(u));
      reinterpret_cast<bf16*>(out)[(size_t)token * pair_offset + col] =
          __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
    } else {
      const int col = n0 + row;
      if (col >= n) continue;
      if (EPI == EPI_SOFTCAP) {
        const float z = __bfloat162float(__float2bfloat16_rn(v)) * multiplier;
        reinterpret_cast<float*>(out)[(size_t)token * n + col] = cap > 0.f ? cap * tanhf(z / cap) : z;
      } else {
        reinterpret_cast<bf16*>(out)[(size_t)token * n + col] = __float2bfloat16_rn(v);
      }
    }
  }
}

template <int NT, int RG, int EPI, int WARPS>
int launch_warps(int blocks, const bf16* a, const bf16* w, void* out, int m, int n, int k, int pair_offset,
                 float multiplier, float cap, cudaStream_t stream) {
  constexpr size_t smem = sizeof(float) * WARPS * RG * 16 * (NT * 8 + 1);
  static bool configured = false;
  if (smem > 48 * 1024 && !configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<NT, RG, EPI, WARPS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  launch_pdl(gemm_skinny_kernel<NT, RG, EPI, WARPS>, blocks, WARPS * 32, smem, stream, a, w, out, m, n, k, pair_offset,
             multiplier, cap);
  return OMNIA_LAUNCH_RESULT();
}

template <int NT, int RG, int EPI>
int launch_variant(int blocks, const bf16* a, const bf16* w, void* out, int m, int n, int k, int pair_offset,
                   float multiplier, float cap, cudaStream_t stream) {
  // A grid of at most one wave leaves every block a long slice of k: sixteen warps halve it.
  if (NT <= 2 && blocks <= omnia_sm_count())
    return launch_warps<NT, RG, EPI, 16>(blocks, a, w, out, m, n, k, pair_offset, multiplier, cap, stream);
  return launch_warps<NT, RG, EPI, 8>(blocks, a, w, out, m, n, k, pair_offset, multiplier, cap, stream);
}

template <int NT, int EPI>
int launch(const bf16* a, const bf16* w, void* out, int m, int n, int k, int pair_offset,
           float multiplier, float cap, cudaStream_t stream) {
  if (EPI == EPI_SWIGLU)
    return launch_variant<NT, 2, EPI>((pair_offset + 15) / 16, a, w, out, m, n, k, pair_offset, multiplier, cap, stream);
  if (NT <= 2 && n >= 32 * omnia_sm_count())
    return launch_variant<NT, 2, EPI>((n + 31) / 32, a, w, out, m, n, k, 0, multiplier, cap, stream);
  return launch_variant<NT, 1, EPI>((n + 15) / 16, a, w, out, m, n, k, 0, multiplier, cap, stream);
}

template <int EPI>
int launch_rows(const bf16* a, const bf16* w, void* out, int m, int n, int k, int pair_offset, float multiplier,
                float cap, cudaStream_t stream) {
  if (m <= 8) return launch<1, EPI>(a, w, out, m, n, k, pair_offset, multiplier, cap, stream);
  if (m <= 16) return launch<2, EPI>(a, w, out, m, n, k, pair_offset, multiplier, cap, stream);
  if (m <= 32) return launch<4, EPI>(a, w, out, m, n, k, pair_offset, multiplier, cap, stream);
  return launch<8, EPI>(a, w, out, m, n, k, pair_offset, multiplier, cap, stream);
}

}  // namespace

// epilogue: 0 store bfloat16 [m, n]; 1 SwiGLU, w = [gate rows | up rows] with n = 2 * inner,
// out bfloat16 [m, inner]; 2 soft cap, out float32 [m, n].
extern "C" int omnia_gemm_skinny(const void* a, const void* w, void* out, int m, int n, int k,
                                 int epilogue, float multiplier, float cap, cudaStream_t stream) {
  if (m == 0 || n == 0) return 0;
  if (m > 64 || k % 8 != 0 || k <= 0) return (int)cudaErrorInvalidValue;
  const bf16* ap = (const bf16*)a;
  const bf16* wp = (const bf16*)w;
  if (epilogue == EPI_SWIGLU) {
    if (n % 2) return (int)cudaErrorInvalidValue;
    return launch_rows<EPI_SWIGLU>(ap, wp, out, m, n, k, n / 2, 1.f, 0.f, stream);
  }
  if (epilogue == EPI_SOFTCAP) return launch_rows<EPI_SOFTCAP>(ap, wp, out, m, n, k, 0, multiplier, cap, stream);
  if (epilogue != EPI_STORE) return (int)cudaErrorInvalidValue;
  return launch_rows<EPI_STORE>(ap, wp, out, m, n, k, 0, 1.f, 0.f, stream);
}
