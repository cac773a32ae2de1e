// out[m, n] = sum_k a[m, k] * w[n, k] for up to 16 rows m (decode steps), the weight matrix
// streamed from HBM exactly once through a ring in shared memory.
//
// One block per SM owns a contiguous run of 16-row tiles of the matrix. A producer warp copies
// the tiles into the ring with TMA, boxes of 8 rows x 256 columns (4 KB), 1024 columns of a tile
// (32 KB) per stage, four stages, signalled by mbarriers. Measured on B200 while tuning this:
// a stage costs about half a microsecond to hand over whatever its size, so stages of 16 KB
// reach 4.3 TB/s and stages of 32 KB 6.8 TB/s with the same bytes in flight; rows copied one by
// one (1 KB bulk copies) reach 2.6 TB/s. The weights never depend on the kernel before this
// one, so the producer starts at once (the launch is a programmatic dependent launch) and only
// the eight consumer warps wait for the activations. Each consumer warp takes 128 columns of
// every stage, builds m16n8k16 fragments from 16-byte reads (a dot product does not care about
// the order of k, so eight consecutive k of a weight row meet the same eight k of an activation
// row and no shuffle is needed), and the warps' partial sums of a tile are added through shared
// memory in a fixed order: results do not depend on timing. Activations are fetched from L2 one
// stage ahead into registers.
//
// Epilogues: plain store; SwiGLU (a tile is eight gate rows over the eight up rows of the same
// columns, and the block stores silu(gate) * up); soft cap (float32 logits).
// bfloat16 operands, float32 accumulation; k a multiple of 8; a, w 16-byte aligned.
//
// A residual step that is still pending can ride along (PENDING): instead of activations the kernel
// is given the float32 residual x, the branch that is to be added to it and the two norms' weights,
//   x_out = x + rms(branch) * wb,   a = bfloat16(rms(x_out) * wo),
// and every block works this out for itself while its first weights are on their way: a consumer
// warp takes a row (hence at most eight), a lane holds its 1/32 of the row in registers (hence at
// most 2,048 columns), the normalised row goes to shared memory, where the activations
// are then fetched from, and one block per row writes x_out. x is not updated in place: other
// blocks are still reading it.
//
// Every wait on a barrier is bounded: when the bound is hit the block raises OMNIA_ERR_TIMEOUT
// in the error word, its warps leave their loops, the producer waits (bounded again) for the
// copies it still has in flight, and the block returns.
#include <cuda.h>

#include "common.cuh"

#define OMNIA_ERR_TIMEOUT 8

#ifndef GEMV_STAGES
#define GEMV_STAGES 4
#endif

namespace {

typedef __nv_bfloat16 bf16;

constexpr int CONSUMER_WARPS = 8;
constexpr int CONSUMERS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMERS + 32;
constexpr int TILE_ROWS = 16;
#ifndef GEMV_WARP_COLS
#define GEMV_WARP_COLS 128
#endif
constexpr int WARP_COLS = GEMV_WARP_COLS;                  // columns of a stage per consumer warp (a multiple of 32)
constexpr int KBLOCKS = WARP_COLS / 32;                    // 32-column steps of a warp per stage
constexpr int STAGE_COLS = CONSUMER_WARPS * WARP_COLS;     // 1024
constexpr int BOX_ROWS = 8, BOX_COLS = 256;                // one TMA copy; lands dense, [8][256]
constexpr int BOX_BYTES = BOX_ROWS * BOX_COLS * 2;
constexpr int BOXES_ACROSS = STAGE_COLS / BOX_COLS;        // boxes side by side in a stage
constexpr int STAGE_BOXES = 2 * BOXES_ACROSS;              // upper eight rows, then lower eight rows
constexpr int STAGE_BYTES = STAGE_BOXES * BOX_BYTES;
static_assert(STAGE_COLS % BOX_COLS == 0 && STAGE_BOXES <= 32, "a stage is at most 32 boxes");
constexpr int STAGES = GEMV_STAGES;
#ifndef GEMV_GROUP_TILES
#define GEMV_GROUP_TILES 4
#endif
constexpr int GROUP_TILES = GEMV_GROUP_TILES;              // tiles that share one fetch of the activations
constexpr uint32_t WAIT_LIMIT = 1u << 20;

enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_SOFTCAP = 2 };

// A pending residual step (see the head of the file). wb / wo null: a norm without weights;
// norm_branch 0: the branch is added as it is.
struct PendingStep {
  const float* x;
  float* x_out;
  const bf16* branch;
  const float* wb;
  const float* wo;
  float eps_b, eps_o;
  int norm_branch;
};
constexpr int PENDING_MAX_K = 2048;                        // a lane holds k / 32 values of a row
constexpr int PENDING_CHUNKS = PENDING_MAX_K / (32 * 8);   // 8-column chunks of a row per lane
constexpr int PENDING_PAD = 8;                             // columns between the rows in shared memory

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
// Bounded wait; false when the block is giving up (its own limit, or another warp's).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (omnia_mbar_test(bar, parity)) return true;
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try(bar, parity)) return true;
    if ((i & 63) == 63 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void mma_bf16(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory"); }

// The matrix row that row r (0..15) of tile `tile` holds, or -1 when it lies outside the matrix.
template <int EPI>
__device__ __forceinline__ int tile_row(int tile, int r, int n, int inner) {
  if (EPI == EPI_SWIGLU) {
    const int col = tile * 8 + (r & 7);
    return col < inner ? (r < 8 ? col : inner + col) : -1;
  }
  const int row = tile * TILE_ROWS + r;
  return row < n ? row : -1;
}

// NT: activation tiles of 8 rows (1 for m <= 8, 2 for m <= 16).
__host__ __device__ constexpr size_t partial_bytes(int nt) { return sizeof(float) * CONSUMER_WARPS * GROUP_TILES * TILE_ROWS * (nt * 8 + 1); }

template <int NT, int EPI, bool PENDING>
__global__ void __launch_bounds__(THREADS, 1)
gemv_stream_kernel(const bf16* __restrict__ a, const __grid_constant__ CUtensorMap map_w, void* __restrict__ out,
                   int m, int n, int k, int inner, int tiles, float multiplier, float cap, const PendingStep pending,
                   int* __restrict__ err) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* ring = smem;
  float (*partial)[GROUP_TILES * TILE_ROWS][NT * 8 + 1] =
      reinterpret_cast<float (*)[GROUP_TILES * TILE_ROWS][NT * 8 + 1]>(smem + STAGES * STAGE_BYTES);
  // PENDING: the normalised rows, [NT * 8][k + PENDING_PAD] bfloat16.
  bf16* normed = reinterpret_cast<bf16*>(smem + STAGES * STAGE_BYTES + ((partial_bytes(NT) + 15) & ~(size_t)15));
  // PENDING: the two norms' weights, [2][k] float32 (ones where a norm has none).
  float* norm_w = reinterpret_cast<float*>(normed + (size_t)NT * 8 * (k + PENDING_PAD));
  __shared__ __align__(8) unsigned long long bars[2 * STAGES];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, CONSUMER_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // This block's tiles: a contiguous run, sizes differing by at most one between blocks. They
  // are worked on in groups of GROUP_TILES: for every 1024 columns, the stages of all tiles of
  // the group follow one another, so a warp fetches its activations of those columns once per
  // group (from L2, which is far: fetched per stage they bounded a stage's time from below).
  const int base = tiles / gridDim.x, extra = tiles % gridDim.x;
  const int my_tiles = base + ((int)blockIdx.x < extra ? 1 : 0);
  const int tile0 = blockIdx.x * base + min((int)blockIdx.x, extra);
  const int chunks = (k + STAGE_COLS - 1) / STAGE_COLS;

  if (warp == CONSUMER_WARPS) {
    // ---- producer: needs nothing from the kernel before, so it does not wait for it ----
    int s = 0, phase = 1, in_flight = 0;
    bool ok = true;
    for (int first = 0; first < my_tiles && ok; first += GROUP_TILES) {
      const int count = min(GROUP_TILES, my_tiles - first);
      for (int c = 0; c < chunks && ok; ++c)
        for (int i = 0; i < count; ++i) {
          if (lane == 0) ok = mbar_wait(empty0 + 8 * s, phase, abort_flag);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          const int tile = tile0 + first + i;
          // Lane i copies box i of the stage: half i / BOXES_ACROSS (rows g, then rows g + 8) and
          // 256 columns. A box that starts outside the matrix is not copied (its rows and columns
          // are masked by the consumers); one that straddles an edge is filled with zeros there.
          const int half = lane / BOXES_ACROSS, x = c * STAGE_COLS + (lane % BOXES_ACROSS) * BOX_COLS;
          const int y = lane < STAGE_BOXES ? tile_row<EPI>(tile, half * 8, n, inner) : -1;
          const bool copies = y >= 0 && x < k;
          const unsigned live = __ballot_sync(0xffffffffu, copies);
          if (lane == 0) mbar_expect_tx(full0 + 8 * s, (uint32_t)__popc(live) * BOX_BYTES);
          __syncwarp();
          if (copies) tma_load_2d(smem_u32(ring + s * STAGE_BYTES + lane * BOX_BYTES), &map_w, full0 + 8 * s, x, y);
          in_flight = min(in_flight + 1, STAGES);
          if (++s == STAGES) s = 0, phase ^= 1;
        }
    }
    pdl_launch_dependents();
    if (!ok && lane == 0) {
      // Giving up: the copies already issued must land before the block's shared memory is released.
      // The last `in_flight` stages before s were filled in phase `phase ^ 1` of their barriers, or
      // in phase `phase` when the ring wrapped between them and s.
      for (int back = 1; back <= in_flight; ++back) {
        const int st = (s - back + STAGES) % STAGES;
        const int filled_phase = (st < s ? phase : phase ^ 1) ^ 1;
        for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(full0 + 8 * st, filled_phase); ++i) {
        }
      }
    }
  } else {
    // ---- consumers ----
    const int g = lane >> 2, t = lane & 3;
    const bf16* arow[NT];
    bool alive[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      alive[j] = 8 * j + g < m;
      arow[j] = a + (size_t)(alive[j] ? 8 * j + g : 0) * k;
    }
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const int in_stage = warp * WARP_COLS + 8 * t;  // this thread's first column within a stage
    if (PENDING) {
      // The norms' weights depend on no kernel, and the stream of matrices has long pushed them
      // out of L2: they are fetched before the wait, so that after it only x and the branch are far.
      for (int col = (threadIdx.x) * 4; col < k; col += CONSUMERS * 4) {
        const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
        *reinterpret_cast<float4*>(norm_w + col) =
            pending.norm_branch && pending.wb ? __ldg(reinterpret_cast<const float4*>(pending.wb + col)) : one;
        *reinterpret_cast<float4*>(norm_w + k + col) =
            pending.wo ? __ldg(reinterpret_cast<const float4*>(pending.wo + col)) : one;
      }
      consumer_sync();
    }
    pdl_wait();  // the activations come from the kernel before
    // From here on every earlier kernel is complete, so the next kernel's blocks may move in beside
    // this one (never more than two kernels overlap). Activations are read through L2 (__ldcg): a
    // block that started while an earlier kernel was still running must not find lines in L1 that
    // that kernel's blocks on the same SM left there.
    pdl_launch_dependents();
    if (PENDING) {
      const int stride = k + PENDING_PAD;
#pragma unroll 1
      for (int j = 0; j < NT; ++j) {
        const int row = warp + 8 * j;
        if (row >= m) break;
        const bf16* br = pending.branch + (size_t)row * k;
        const float* xr = pending.x + (size_t)row * k;
        uint4 bv[PENDING_CHUNKS];
        float xn[PENDING_CHUNKS][8];
        // Everything the row needs is asked for at once; the two sums then only wait for it.
#pragma unroll
        for (int i = 0; i < PENDING_CHUNKS; ++i) {
          const int col = (i * 32 + lane) * 8;
          bv[i] = col < k ? __ldcg(reinterpret_cast<const uint4*>(br + col)) : zero;
          const float4 lo = col < k ? __ldcg(reinterpret_cast<const float4*>(xr + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
          const float4 hi = col < k ? __ldcg(reinterpret_cast<const float4*>(xr + col + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
          xn[i][0] = lo.x, xn[i][1] = lo.y, xn[i][2] = lo.z, xn[i][3] = lo.w;
          xn[i][4] = hi.x, xn[i][5] = hi.y, xn[i][6] = hi.z, xn[i][7] = hi.w;
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < PENDING_CHUNKS; ++i) {
          const unsigned w4[4] = {bv[i].x, bv[i].y, bv[i].z, bv[i].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[e]));
            ss += f.x * f.x + f.y * f.y;
          }
        }
        const float scale_b = pending.norm_branch ? rsqrtf(warp_sum(ss) / (float)k + pending.eps_b) : 1.f;
        const bool writes = (int)blockIdx.x == row % (int)gridDim.x;  // one block stores the row's new residual
        ss = 0.f;
#pragma unroll
        for (int i = 0; i < PENDING_CHUNKS; ++i) {
          const int col = (i * 32 + lane) * 8;
          if (col >= k) continue;
          float gb[8];
          {
            const float4 lo = *reinterpret_cast<const float4*>(norm_w + col);
            const float4 hi = *reinterpret_cast<const float4*>(norm_w + col + 4);
            gb[0] = lo.x, gb[1] = lo.y, gb[2] = lo.z, gb[3] = lo.w, gb[4] = hi.x, gb[5] = hi.y, gb[6] = hi.z, gb[7] = hi.w;
          }
          const unsigned w4[4] = {bv[i].x, bv[i].y, bv[i].z, bv[i].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[e]));
            float v0 = f.x, v1 = f.y;
            if (pending.norm_branch) v0 = v0 * scale_b * gb[2 * e], v1 = v1 * scale_b * gb[2 * e + 1];
            xn[i][2 * e] += v0;
            xn[i][2 * e + 1] += v1;
            ss += xn[i][2 * e] * xn[i][2 * e] + xn[i][2 * e + 1] * xn[i][2 * e + 1];
          }
          if (writes) {
            float* dst = pending.x_out + (size_t)row * k + col;
            *reinterpret_cast<float4*>(dst) = make_float4(xn[i][0], xn[i][1], xn[i][2], xn[i][3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(xn[i][4], xn[i][5], xn[i][6], xn[i][7]);
          }
        }
        const float scale_o = rsqrtf(warp_sum(ss) / (float)k + pending.eps_o);
#pragma unroll
        for (int i = 0; i < PENDING_CHUNKS; ++i) {
          const int col = (i * 32 + lane) * 8;
          if (col >= k) continue;
          float go[8];
          {
            const float4 lo = *reinterpret_cast<const float4*>(norm_w + k + col);
            const float4 hi = *reinterpret_cast<const float4*>(norm_w + k + col + 4);
            go[0] = lo.x, go[1] = lo.y, go[2] = lo.z, go[3] = lo.w, go[4] = hi.x, go[5] = hi.y, go[6] = hi.z, go[7] = hi.w;
          }
          uint4 packed;
          packed.x = pack_bf16(xn[i][0] * scale_o * go[0], xn[i][1] * scale_o * go[1]);
          packed.y = pack_bf16(xn[i][2] * scale_o * go[2], xn[i][3] * scale_o * go[3]);
          packed.z = pack_bf16(xn[i][4] * scale_o * go[4], xn[i][5] * scale_o * go[5]);
          packed.w = pack_bf16(xn[i][6] * scale_o * go[6], xn[i][7] * scale_o * go[7]);
          *reinterpret_cast<uint4*>(normed + (size_t)row * stride + col) = packed;
        }
      }
      consumer_sync();  // every warp reads every row
    }
    auto fetch = [&](int c, uint4 (&dst)[KBLOCKS][NT]) {
      const int col0 = c * STAGE_COLS + in_stage;
#pragma unroll
      for (int h = 0; h < KBLOCKS; ++h)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          if (!alive[j] || col0 + 32 * h >= k)
            dst[h][j] = zero;
          else if (PENDING)
            dst[h][j] = *reinterpret_cast<const uint4*>(normed + (size_t)(8 * j + g) * (k + PENDING_PAD) + col0 + 32 * h);
          else
            dst[h][j] = __ldcg(reinterpret_cast<const uint4*>(arow[j] + col0 + 32 * h));
        }
    };
    uint4 av[KBLOCKS][NT], av_next[KBLOCKS][NT];
    if (my_tiles > 0) fetch(0, av_next);
    bool ok = true;
    int s = 0, phase = 0;
    for (int first = 0; first < my_tiles && ok; first += GROUP_TILES) {
      const int count = min(GROUP_TILES, my_tiles - first);
      float acc[GROUP_TILES][NT][4];
#pragma unroll
      for (int i = 0; i < GROUP_TILES; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
      for (int c = 0; c < chunks && ok; ++c) {
#pragma unroll
        for (int h = 0; h < KBLOCKS; ++h)
#pragma unroll
          for (int j = 0; j < NT; ++j) av[h][j] = av_next[h][j];
        // The next columns' activations (the first columns again when another group follows).
        if (c + 1 < chunks || first + GROUP_TILES < my_tiles) fetch(c + 1 < chunks ? c + 1 : 0, av_next);
        const int col0 = c * STAGE_COLS + in_stage;
#pragma unroll
        for (int i = 0; i < GROUP_TILES; ++i) {
          if (i >= count) break;
          const int tile = tile0 + first + i;
          const bool lo_live = tile_row<EPI>(tile, g, n, inner) >= 0, hi_live = tile_row<EPI>(tile, g + 8, n, inner) >= 0;
          ok = mbar_wait(full0 + 8 * s, phase, abort_flag);
          if (!ok) break;
          // Column in_stage + 32 h of the stage: box (that / 256), then rows of 512 bytes.
          static_assert(BOX_COLS % WARP_COLS == 0, "a warp's columns of a stage lie in one box");
          const uint32_t stage = smem_u32(ring + s * STAGE_BYTES) + (in_stage / BOX_COLS) * BOX_BYTES +
                                 g * (BOX_COLS * 2) + (in_stage % BOX_COLS) * 2;
#pragma unroll
          for (int h = 0; h < KBLOCKS; ++h) {
            const bool live = col0 + 32 * h < k;
            uint4 lo = lds128(stage + 64 * h), hi = lds128(stage + 64 * h + BOXES_ACROSS * BOX_BYTES);
            if (!live || !lo_live) lo = zero;
            if (!live || !hi_live) hi = zero;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
              mma_bf16(acc[i][j], lo.x, hi.x, lo.y, hi.y, av[h][j].x, av[h][j].y);
              mma_bf16(acc[i][j], lo.z, hi.z, lo.w, hi.w, av[h][j].z, av[h][j].w);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty0 + 8 * s);  // the stage may be filled again
          if (++s == STAGES) s = 0, phase ^= 1;
        }
      }
      if (!ok) break;

      // The group is complete: add the warps' partial sums in a fixed order and store.
#pragma unroll
      for (int i = 0; i < GROUP_TILES; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          partial[warp][i * TILE_ROWS + g][j * 8 + 2 * t] = acc[i][j][0];
          partial[warp][i * TILE_ROWS + g][j * 8 + 2 * t + 1] = acc[i][j][1];
          partial[warp][i * TILE_ROWS + g + 8][j * 8 + 2 * t] = acc[i][j][2];
          partial[warp][i * TILE_ROWS + g + 8][j * 8 + 2 * t + 1] = acc[i][j][3];
        }
      consumer_sync();
      const int out_rows = EPI == EPI_SWIGLU ? 8 : TILE_ROWS;
      for (int idx = threadIdx.x; idx < count * out_rows * NT * 8; idx += CONSUMERS) {
        const int token = idx / (count * out_rows), rest = idx % (count * out_rows);
        const int i = rest / out_rows, r = rest % out_rows, tile = tile0 + first + i;
        if (token >= m) continue;
        float v = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < CONSUMER_WARPS; ++s2) v += partial[s2][i * TILE_ROWS + r][token];
        if (EPI == EPI_SWIGLU) {
          float up = 0.f;
#pragma unroll
          for (int s2 = 0; s2 < CONSUMER_WARPS; ++s2) up += partial[s2][i * TILE_ROWS + 8 + r][token];
          const int col = tile * 8 + r;
          if (col >= inner) continue;
          // The two halves are rounded to bfloat16 first, as a separate product would round them.
          const float gate = __bfloat162float(__float2bfloat16_rn(v));
          up = __bfloat162float(__float2bfloat16_rn(up));
          reinterpret_cast<bf16*>(out)[(size_t)token * inner + col] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
        } else {
          const int col = tile * TILE_ROWS + r;
          if (col >= n) continue;
          if (EPI == EPI_SOFTCAP) {
            const float z = __bfloat162float(__float2bfloat16_rn(v)) * multiplier;
            reinterpret_cast<float*>(out)[(size_t)token * n + col] = cap > 0.f ? cap * tanhf(z / cap) : z;
          } else {
            reinterpret_cast<bf16*>(out)[(size_t)token * n + col] = __float2bfloat16_rn(v);
          }
        }
      }
      consumer_sync();  // the partial sums are read before the next group overwrites them
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicOr(err, OMNIA_ERR_TIMEOUT);
}

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

// The [rows, k] bfloat16 row-major matrix as a 2-D tensor map with dense boxes of 8 rows x 256 columns;
// what a box covers beyond the matrix is filled with zeros.
bool make_map(CUtensorMap* map, const void* base, int rows, int k) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)k * sizeof(bf16)};
  const cuuint32_t box[2] = {(cuuint32_t)BOX_COLS, (cuuint32_t)BOX_ROWS};
  const cuuint32_t elem[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The most dynamic shared memory a launch of this shape asks for.
template <int NT, bool PENDING>
constexpr size_t fixed_most() {
  return (size_t)STAGES * STAGE_BYTES + ((partial_bytes(NT) + 15) & ~(size_t)15) +
         (PENDING ? sizeof(bf16) * NT * 8 * (size_t)(PENDING_MAX_K + PENDING_PAD) + sizeof(float) * 2 * PENDING_MAX_K : 0);
}

template <int NT, int EPI, bool PENDING>
int launch(const bf16* a, const bf16* w, void* out, int m, int n, int k, int inner, float multiplier, float cap,
           const PendingStep& pending, int* err, cudaStream_t stream) {
  const size_t fixed = (size_t)STAGES * STAGE_BYTES + ((partial_bytes(NT) + 15) & ~(size_t)15);
  const size_t smem = fixed + (PENDING ? sizeof(bf16) * NT * 8 * (size_t)(k + PENDING_PAD) + sizeof(float) * 2 * k : 0);
  constexpr size_t most = fixed_most<NT, PENDING>();
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemv_stream_kernel<NT, EPI, PENDING>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
    if (e != cudaSuccess) {
      sms = 0;
      return (int)e;
    }
  }
  CUtensorMap map_w;
  if (!make_map(&map_w, w, n, k)) return (int)cudaErrorInvalidValue;
  const int tiles = EPI == EPI_SWIGLU ? (inner + 7) / 8 : (n + TILE_ROWS - 1) / TILE_ROWS;
  launch_pdl(gemv_stream_kernel<NT, EPI, PENDING>, min(tiles, sms), THREADS, smem, stream, a, map_w, out, m, n, k, inner,
             tiles, multiplier, cap, pending, err);
  return OMNIA_LAUNCH_RESULT();
}

template <int EPI, bool PENDING>
int launch_rows(const bf16* a, const bf16* w, void* out, int m, int n, int k, int inner, float multiplier, float cap,
                const PendingStep& pending, int* err, cudaStream_t stream) {
  if (m <= 8) return launch<1, EPI, PENDING>(a, w, out, m, n, k, inner, multiplier, cap, pending, err, stream);
  if (PENDING) return (int)cudaErrorInvalidValue;  // sixteen normalised rows and the weights do not fit beside the ring
  return launch<2, EPI, false>(a, w, out, m, n, k, inner, multiplier, cap, pending, err, stream);
}

}  // namespace

// epilogue: 0 store bfloat16 [m, n]; 1 SwiGLU, w = [gate rows | up rows] with n = 2 * inner,
// out bfloat16 [m, inner]; 2 soft cap, out float32 [m, n]. err: the device error word.
extern "C" int omnia_gemv_stream(const void* a, const void* w, void* out, int m, int n, int k, int epilogue,
                                 float multiplier, float cap, int* err, cudaStream_t stream) {
  if (m == 0 || n == 0) return 0;
  if (m > 16 || k % 8 != 0 || k <= 0) return (int)cudaErrorInvalidValue;
  if (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) != 0) return (int)cudaErrorInvalidValue;
  const bf16* ap = (const bf16*)a;
  const bf16* wp = (const bf16*)w;
  const PendingStep none{};
  if (epilogue == EPI_SWIGLU) {
    if (n % 2) return (int)cudaErrorInvalidValue;
    return launch_rows<EPI_SWIGLU, false>(ap, wp, out, m, n, k, n / 2, 1.f, 0.f, none, err, stream);
  }
  if (epilogue == EPI_SOFTCAP)
    return launch_rows<EPI_SOFTCAP, false>(ap, wp, out, m, n, k, 0, multiplier, cap, none, err, stream);
  if (epilogue != EPI_STORE) return (int)cudaErrorInvalidValue;
  return launch_rows<EPI_STORE, false>(ap, wp, out, m, n, k, 0, 1.f, 0.f, none, err, stream);
}

extern "C" int omnia_gemv_stream_pending_max_k(void) { return PENDING_MAX_K; }

// The same product with a pending residual step in front of it (epilogues 0 and 1):
//   x_out = x + (norm_branch ? rms(branch, eps_b) * wb : branch),  a = bfloat16(rms(x_out, eps_o) * wo),
// x, x_out float32 [m, k] (different buffers, m <= 8), branch bfloat16 [m, k], wb, wo float32 [k] or null.
extern "C" int omnia_gemv_stream_pending(const float* x, float* x_out, const void* branch, const float* wb,
                                         float eps_b, int norm_branch, const float* wo, float eps_o, const void* w,
                                         void* out, int m, int n, int k, int epilogue, int* err,
                                         cudaStream_t stream) {
  if (m == 0 || n == 0) return 0;
  if (m > 8 || k % 8 != 0 || k <= 0 || k > PENDING_MAX_K || x == x_out) return (int)cudaErrorInvalidValue;
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(x_out) | reinterpret_cast<uintptr_t>(branch) |
        reinterpret_cast<uintptr_t>(wb) | reinterpret_cast<uintptr_t>(wo) | reinterpret_cast<uintptr_t>(w)) & 15) != 0)
    return (int)cudaErrorInvalidValue;
  const PendingStep pending{x, x_out, (const bf16*)branch, wb, wo, eps_b, eps_o, norm_branch};
  const bf16* wp = (const bf16*)w;
  if (epilogue == EPI_SWIGLU) {
    if (n % 2) return (int)cudaErrorInvalidValue;
    return launch_rows<EPI_SWIGLU, true>(nullptr, wp, out, m, n, k, n / 2, 1.f, 0.f, pending, err, stream);
  }
  if (epilogue != EPI_STORE) return (int)cudaErrorInvalidValue;
  return launch_rows<EPI_STORE, true>(nullptr, wp, out, m, n, k, 0, 1.f, 0.f, pending, err, stream);
}
