// out[m, n] = sum_k a[m, k] * w[n, k] in bfloat16 on the 5th-generation tensor cores, two SMs to a
// tile (tcgen05 cta_group::2): a cluster of two blocks owns a 256 x 256 tile of the output. Each
// block stages its own 128 rows of a and its own half (128 rows) of the w tile by TMA, so a block
// brings in 32 KB per step of k = 64 where a block that owns a 128 x 256 tile alone brings 48 KB: at
// 1.1 PFLOP/s the one-block kernel pulls about 12 TB/s of operands out of L2, which is what bounds it.
// The leader block (cluster rank 0) issues every MMA for the pair; the instruction reads a's rows
// from each block's own shared memory, the two halves of w from both, and writes each block's 128
// rows of the accumulator into that block's own tensor memory.
//   warp 0   producer (both blocks): waits for a free stage, issues its two TMA loads; they count
//            on the leader's "full" barrier of the stage (the leader arms it with both blocks' bytes)
//   warp 1   allocates tensor memory (both blocks); in the leader its elected lane waits for a
//            drained accumulator, issues four MMAs per full stage, and tcgen05.commit (multicast to
//            both blocks) frees the stage in both and, after the last step, signals "accumulator full"
//   warps 2-5  (both blocks) read their block's 128 accumulator rows, apply the epilogue, store, and
//            arrive on the leader's "accumulator empty" barrier
// Blocks are persistent (one per SM); clusters take tiles round-robin; two accumulators in tensor
// memory let the epilogue of one tile run while the next is multiplied. Epilogues: 0 store
// bfloat16; 1 SwiGLU: the leader stages 128 gate rows of w, its peer the matching 128 up rows, the
// blocks store silu(gate) * up; 2 soft cap to float32; 3 the attention input projection
// [q | gate | k | v]: a tile's 256 columns are whole heads, and the thread that owns a row gives each
// head of q and k its weightless RMS norm and its rotation (angles from a table of the step's
// positions), stores q to [tokens, heads, head size] and k and v straight into the cache pages at
// the row's slot; columns of neither (the gate) are stored as epilogue 0 does.
//
// Every wait on a barrier is bounded: when the bound is hit the block raises OMNIA_ERR_TIMEOUT in
// the error word and its roles leave their loops (its peer's waits then run out too); both blocks
// meet at the cluster barrier, free their tensor memory and return.
#include <cuda.h>

#include "common.cuh"

#define OMNIA_ERR_TIMEOUT 8

namespace {

typedef __nv_bfloat16 bf16;

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;   // 128 bytes of bfloat16: one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;  // producer warp, MMA warp, four epilogue warps
constexpr uint32_t WAIT_LIMIT = 1u << 20;

enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_SOFTCAP = 2, EPI_QKV = 3 };

// What epilogue 3 needs besides the product's own arguments.
struct QkvParts {
  int head_dim, q_col, k_col, v_col, nq, nkv;  // q: columns [q_col, q_col + nq * head_dim); k and v alike with nkv
  float eps;                                    // of the norm of q and k heads; < 0: no norm
  const float2* angles;                         // [head_dim / 2, rows] (cos, sin) at each row's position; null: no rotation
  const long long* slots;                       // [rows] the cache slot of each row (negative: not stored); null with nkv 0
  bf16* q_out;                                  // [rows, nq, head_dim]
  bf16* pages;                                  // [pages, 2, nkv, page_size, head_dim]
  int page_size;
  long long num_slots;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (omnia_mbar_test(bar, parity)) return true;
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try(bar, parity)) return true;
    if ((i & 63) == 63 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}


// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes,
// eight-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);  // start address
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                       // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
  return d;
}

// kind::f16 instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
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


constexpr int STAGES = 6;
// The accumulator's columns, TILE_N, are 256 or 192 (a template parameter): the narrower tile is for
// shapes whose 256-wide tiles leave the last wave of clusters mostly idle (12,288 columns of
// gate|up at 2,048 rows: 384 tiles on 74 clusters are six waves, the last with 14 tiles; 512 tiles of
// 192 are seven waves of three quarters the length). Each block stages TILE_N / 2 rows of w.
constexpr uint32_t A_BYTES = BLOCK_M * BLOCK_K * sizeof(bf16);
constexpr uint32_t ACC_STRIDE = 256;                                // tensor-memory columns between the two accumulators
constexpr uint32_t TMEM_COLS = 512;                                 // a power of two, as allocations must be

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, of `addr` in the block of rank `rank`.
__device__ __forceinline__ uint32_t in_block(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A TMA load whose bytes count on a barrier that may stand in the peer block.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this address in both blocks of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((unsigned short)3)
               : "memory");
}

constexpr int ACC_BUFS = 2;                                         // the tile being multiplied, the tile being stored

// Which column of 256-wide tiles the `index`-th one to be worked on is. Epilogue 3 takes the tiles of
// q and k first: theirs is the long epilogue, and the last tiles' epilogues overlap no product.
template <int EPI>
__device__ __forceinline__ int tile_column(int index, const QkvParts& parts) {
  if (EPI != EPI_QKV) return index;
  const int heads = 256 / parts.head_dim;  // of a tile
  if (parts.q_col % 256 || parts.k_col % 256 || parts.nq % heads || parts.nkv % heads) return index;
  const int q_tiles = parts.nq / heads, k_tiles = parts.nkv / heads, q0 = parts.q_col / 256, k0 = parts.k_col / 256;
  if (index < q_tiles) return q0 + index;
  if (index < q_tiles + k_tiles) return k0 + index - q_tiles;
  // The others in their own order: count on past the two ranges, the lower one first.
  int column = index - q_tiles - k_tiles;
  const bool q_first = q0 < k0;
  if (column >= (q_first ? q0 : k0)) column += q_first ? q_tiles : k_tiles;
  if (column >= (q_first ? k0 : q0)) column += q_first ? k_tiles : q_tiles;
  return column;
}

template <int EPI, uint32_t TILE_N>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         void* __restrict__ out, int m, int n, int k, int pair_offset, float multiplier,
                         float cap, int m_tiles, int n_tiles, const QkvParts parts, int* err) {
  constexpr int TILE_COLS = EPI == EPI_SWIGLU ? TILE_N / 2 : TILE_N;
  constexpr uint32_t HALF_N = TILE_N / 2;                           // rows of w a block stages
  constexpr uint32_t B_BYTES = HALF_N * BLOCK_K * sizeof(bf16);
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static_assert(TILE_N % 32 == 0 && TILE_N <= ACC_STRIDE && STAGE_BYTES % 1024 == 0, "tile width");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
  // bars: [0, S) stage full (used in the leader), [S, 2S) stage empty, [2S, 2S+2) accumulator full,
  // [2S+2, 2S+4) accumulator empty (used in the leader)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1, clusters = gridDim.x >> 1;
  const int k_blocks = (k + BLOCK_K - 1) / BLOCK_K;
  const int total_tiles = m_tiles * n_tiles;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const uint32_t acc_full0 = smem_u32(bars + 2 * STAGES), acc_empty0 = smem_u32(bars + 2 * STAGES + 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);   // the leader's producer arms it; both blocks' bytes complete it
      mbar_init(empty0 + 8 * s, 1);  // the leader's commit, multicast
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);   // the leader's commit, multicast
      mbar_init(acc_empty0 + 8 * b, 8);  // one arrival per epilogue warp of either block
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;
  // Everything so far needed nothing from the kernel before this one and ran while it finished
  // (the launch is a programmatic dependent launch); from here on its results are read.
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ---- producer (both blocks) -------------------------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += clusters) {
        const int m0 = (tile % m_tiles) * 2 * BLOCK_M + rank * BLOCK_M, n0 = tile_column<EPI>(tile / m_tiles, parts) * TILE_COLS;
        const int w_row = EPI == EPI_SWIGLU ? (leader ? n0 : pair_offset + n0) : n0 + (int)rank * (int)HALF_N;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t a_dst = smem_u32(tiles + s * STAGE_BYTES), b_dst = a_dst + A_BYTES;
          const uint32_t bar = in_block(full0 + 8 * s, 0);
          if (leader) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
          tma_load_2d_pair(a_dst, &map_a, bar, kb * BLOCK_K, m0);
          tma_load_2d_pair(b_dst, &map_b, bar, kb * BLOCK_K, w_row);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (the leader) --------------------------------------------------------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc(2 * BLOCK_M, TILE_N);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += clusters, ++local) {
        const uint32_t buf = local % ACC_BUFS, round = local / ACC_BUFS;
        ok = mbar_wait(acc_empty0 + 8 * buf, (round & 1) ^ 1, abort_flag);  // both epilogues have drained it
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + buf * ACC_STRIDE;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(full0 + 8 * s, (it / STAGES) & 1, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk) {
            const uint64_t a_desc = umma_desc(a_addr + kk * UMMA_K * sizeof(bf16));
            const uint64_t b_desc = umma_desc(b_addr + kk * UMMA_K * sizeof(bf16));
            umma_pair(acc, a_desc, b_desc, idesc, (kb | kk) != 0);
          }
          umma_commit_pair(empty0 + 8 * s);  // the stage is free in both blocks once these MMAs have read it
        }
        if (ok) umma_commit_pair(acc_full0 + 8 * buf);
      }
    }
  } else {
    // ---- epilogue (both blocks; warps 2..5 own accumulator rows 32 * (warp % 4) .. + 31) ----------
    const int quarter = warp & 3;
    uint32_t local = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < total_tiles && ok; tile += clusters, ++local) {
      const int m0 = (tile % m_tiles) * 2 * BLOCK_M + rank * BLOCK_M, n0 = tile_column<EPI>(tile / m_tiles, parts) * TILE_COLS;
      const int row = m0 + quarter * 32 + lane;
      const uint32_t buf = local % ACC_BUFS, round = local / ACC_BUFS;
      ok = mbar_wait(acc_full0 + 8 * buf, round & 1, abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_base = tmem_base + buf * ACC_STRIDE + ((uint32_t)(quarter * 32) << 16);
      if (EPI == EPI_SWIGLU) {
        bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)row * pair_offset + n0;
#pragma unroll 1
        for (int c = 0; c < (int)TILE_N / 2; c += 32) {
          uint32_t gate[32], up[32];
          tmem_load32(lane_base + c, gate);
          tmem_load32(lane_base + TILE_N / 2 + c, up);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (row < m) {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float v[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                // Both halves are rounded to bfloat16 first, as a separate product would round them.
                const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gate[j + e])));
                const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(up[j + e])));
                v[e] = __fdividef(g, 1.f + __expf(-g)) * u;
              }
              const int col = n0 + c + j;
              if (col + 1 < pair_offset && (pair_offset & 1) == 0) {
                *reinterpret_cast<__nv_bfloat162*>(dst + c + j) = __floats2bfloat162_rn(v[0], v[1]);
              } else {
                if (col < pair_offset) dst[c + j] = __float2bfloat16_rn(v[0]);
                if (col + 1 < pair_offset) dst[c + j + 1] = __float2bfloat16_rn(v[1]);
              }
            }
          }
        }
      } else if (EPI == EPI_QKV) {
        const int d = parts.head_dim, half = d / 2;
        const bool live = row < m;
        const long long slot = live && parts.slots != nullptr ? parts.slots[row] : -1;
        // The accumulator's values rounded to bfloat16 first, as a separate product would store them.
        auto rounded = [](uint32_t bits) { return __bfloat162float(__float2bfloat16_rn(__uint_as_float(bits))); };
        auto store32 = [](bf16* to, const float* v) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]), p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
            *reinterpret_cast<uint4*>(to + j) = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                                                           *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
          }
        };
#pragma unroll 1
        for (int seg = 0; seg < (int)TILE_N && n0 + seg < n; seg += d) {
          const int col0 = n0 + seg;
          // Whose head this is: 0 q, 1 k, 2 v, 3 neither. (The same for every thread of the block.)
          int kind = 3, head = 0;
          if (col0 >= parts.q_col && col0 < parts.q_col + parts.nq * d) kind = 0, head = (col0 - parts.q_col) / d;
          else if (col0 >= parts.k_col && col0 < parts.k_col + parts.nkv * d) kind = 1, head = (col0 - parts.k_col) / d;
          else if (col0 >= parts.v_col && col0 < parts.v_col + parts.nkv * d) kind = 2, head = (col0 - parts.v_col) / d;
          // A slot past the pool is reported (once a row: by whoever has the first head of k) and not stored to.
          if (live && kind == 1 && head == 0 && slot >= parts.num_slots) atomicOr(err, OMNIA_ERR_SLOT);
          bf16* dst = nullptr;
          if (live) {
            if (kind == 0) {
              dst = parts.q_out + ((size_t)row * parts.nq + head) * d;
            } else if (kind == 3) {
              dst = reinterpret_cast<bf16*>(out) + (size_t)row * n + col0;
            } else if (slot >= 0 && slot < parts.num_slots) {
              const long long page = slot / parts.page_size, off = slot % parts.page_size;
              dst = parts.pages + (((page * 2 + (kind == 2)) * parts.nkv + head) * parts.page_size + off) * d;
            }
          }
          float scale = 1.f;
          if (kind <= 1 && parts.eps >= 0.f) {
            float ss[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
            for (int c = 0; c < d; c += 32) {
              uint32_t acc[32];
              tmem_load32(lane_base + seg + c, acc);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float v = rounded(acc[j]);
                ss[j & 3] = fmaf(v, v, ss[j & 3]);
              }
            }
            scale = rsqrtf(((ss[0] + ss[1]) + (ss[2] + ss[3])) / (float)d + parts.eps);
          }
          if (kind <= 1 && parts.angles != nullptr) {
            // Dims i and i + half turn together by the row's angle i.
            const float2* angle = parts.angles + (live ? row : 0);  // this row's column of the table
#pragma unroll 1
            for (int c = 0; c < half; c += 32) {
              uint32_t lo[32], hi[32];
              tmem_load32(lane_base + seg + c, lo);
              tmem_load32(lane_base + seg + half + c, hi);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
              float out_lo[32], out_hi[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float2 turn = __ldg(angle + (size_t)(c + j) * m);  // (cos, sin)
                const float a0 = rounded(lo[j]) * scale, b0 = rounded(hi[j]) * scale;
                out_lo[j] = a0 * turn.x - b0 * turn.y, out_hi[j] = a0 * turn.y + b0 * turn.x;
              }
              if (dst != nullptr) {
                store32(dst + c, out_lo);
                store32(dst + half + c, out_hi);
              }
            }
          } else {
#pragma unroll 1
            for (int c = 0; c < d; c += 32) {
              uint32_t acc[32];
              tmem_load32(lane_base + seg + c, acc);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
              float v[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = rounded(acc[j]) * scale;
              if (dst != nullptr) store32(dst + c, v);
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < (int)TILE_N; c += 32) {
          uint32_t acc[32];
          tmem_load32(lane_base + c, acc);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (row >= m) continue;
          if (EPI == EPI_SOFTCAP) {
            float* dst = reinterpret_cast<float*>(out) + (size_t)row * n + n0 + c;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (n0 + c + j >= n) break;
              const float z = __bfloat162float(__float2bfloat16_rn(__uint_as_float(acc[j]))) * multiplier;
              dst[j] = cap > 0.f ? cap * tanhf(z / cap) : z;
            }
          } else {
            bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)row * n + n0 + c;
            if (n0 + c + 32 <= n && (n & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 packed;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1]));
                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(acc[j + 2]), __uint_as_float(acc[j + 3]));
                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(acc[j + 4]), __uint_as_float(acc[j + 5]));
                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(acc[j + 6]), __uint_as_float(acc[j + 7]));
                packed.x = *reinterpret_cast<uint32_t*>(&p0);
                packed.y = *reinterpret_cast<uint32_t*>(&p1);
                packed.z = *reinterpret_cast<uint32_t*>(&p2);
                packed.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst + j) = packed;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + c + j < n) dst[j] = __float2bfloat16_rn(__uint_as_float(acc[j]));
            }
          }
        }
      }
      // This warp has read its rows of the accumulator: tell the leader's MMA warp.
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(in_block(acc_empty0 + 8 * buf, 0));
    }
  }

  // ---- teardown: the pair meets (nobody's shared or tensor memory goes away under its peer), then
  // the allocating warps free the tensor memory ------------------------------------------------
  if (*abort_flag)  // giving up: let the loads already issued land before the blocks' memory goes away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(err, OMNIA_ERR_TIMEOUT);
}

// ---- host side ---------------------------------------------------------------------------

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

// A [rows, k] bfloat16 row-major matrix as a 2-D tensor map with boxes of 64 x box_rows, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)k * sizeof(bf16)};
  const cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


int sm_count() { return omnia_sm_count(); }

// Tiles of the output for accumulators of `tile_n` columns.
template <int EPI>
long long tile_count(int m, int n, int pair_offset, int tile_n, int* m_tiles, int* n_tiles) {
  const int cols = EPI == EPI_SWIGLU ? pair_offset : n;
  const int tile_cols = EPI == EPI_SWIGLU ? tile_n / 2 : tile_n;
  *n_tiles = (cols + tile_cols - 1) / tile_cols;
  *m_tiles = (m + 2 * BLOCK_M - 1) / (2 * BLOCK_M);
  return (long long)*n_tiles * *m_tiles;
}

template <int EPI, uint32_t TILE_N>
int launch_width(const void* a, const void* w, void* out, int m, int n, int k, int pair_offset, float multiplier,
                 float cap, const QkvParts& parts, int* err, cudaStream_t stream) {
  constexpr uint32_t STAGE_BYTES = A_BYTES + (TILE_N / 2) * BLOCK_K * sizeof(bf16);
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, a, m, k, BLOCK_M) || !make_map(&map_b, w, n, k, (int)(TILE_N / 2)))
    return (int)cudaErrorInvalidValue;
  constexpr size_t smem = (size_t)STAGES * STAGE_BYTES + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI, TILE_N>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int m_tiles, n_tiles;
  const long long total = tile_count<EPI>(m, n, pair_offset, (int)TILE_N, &m_tiles, &n_tiles);
  const int pairs = sm_count() / 2;
  const int clusters = (int)(total < pairs ? total : pairs);  // one persistent block per SM
  launch_pdl(gemm_tcgen05_pair_kernel<EPI, TILE_N>, 2 * clusters, THREADS, smem, stream,
             map_a, map_b, out, m, n, k, pair_offset, multiplier, cap, m_tiles, n_tiles, parts, err);
  return OMNIA_LAUNCH_RESULT();
}

// The width whose waves of tiles take the least time: waves x width, 256 on a tie.
template <int EPI>
int launch(const void* a, const void* w, void* out, int m, int n, int k, int pair_offset, float multiplier,
           float cap, int* err, cudaStream_t stream) {
  const QkvParts parts = {};
  const int pairs = sm_count() / 2;
  int mt, nt;
  const long long wide = (tile_count<EPI>(m, n, pair_offset, 256, &mt, &nt) + pairs - 1) / pairs * 256;
  const long long narrow = (tile_count<EPI>(m, n, pair_offset, 192, &mt, &nt) + pairs - 1) / pairs * 192;
  if (narrow < wide) return launch_width<EPI, 192>(a, w, out, m, n, k, pair_offset, multiplier, cap, parts, err, stream);
  return launch_width<EPI, 256>(a, w, out, m, n, k, pair_offset, multiplier, cap, parts, err, stream);
}

}  // namespace

// epilogue: 0 store bfloat16 [m, n]; 1 SwiGLU, w = [gate rows | up rows] with n = 2 * inner,
// out bfloat16 [m, inner]; 2 soft cap, out float32 [m, n]. a and w must be 16-byte aligned and
// k a multiple of 8 (rows of both matrices start on 16 bytes).
extern "C" int omnia_gemm_tcgen05_pair(const void* a, const void* w, void* out, int m, int n, int k, int epilogue,
                                       float multiplier, float cap, int* err, cudaStream_t stream) {
  if (m == 0 || n == 0) return 0;
  if (k <= 0 || k % 8 != 0 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return (int)cudaErrorInvalidValue;
  if (epilogue == EPI_SWIGLU) {
    if (n % 2) return (int)cudaErrorInvalidValue;
    return launch<EPI_SWIGLU>(a, w, out, m, n, k, n / 2, 1.f, 0.f, err, stream);
  }
  if (epilogue == EPI_SOFTCAP) return launch<EPI_SOFTCAP>(a, w, out, m, n, k, 0, multiplier, cap, err, stream);
  if (epilogue != EPI_STORE) return (int)cudaErrorInvalidValue;
  return launch<EPI_STORE>(a, w, out, m, n, k, 0, 1.f, 0.f, err, stream);
}

// The attention input projection with epilogue 3: out [m, n] receives the columns that are neither
// q, k nor v (the gate's); q_out [m, nq, head_dim]; k and v go to pages [.., 2, nkv, page_size,
// head_dim] at slots[row] (nkv 0: nothing is stored). head_dim 64 or 128; q_col, k_col, v_col and n
// multiples of head_dim, so that every head_dim columns of a tile are one head of one kind; angles
// [head_dim / 2, m] (cos, sin) or null; eps < 0: no norm.
extern "C" int omnia_gemm_tcgen05_pair_qkv(const void* a, const void* w, void* out, int m, int n, int k, int head_dim,
                                           int q_col, int k_col, int v_col, int nq, int nkv, float eps,
                                           const void* angles, const long long* slots, void* q_out, void* pages,
                                           int page_size, long long num_slots, int* err, cudaStream_t stream) {
  if (m == 0 || n == 0) return 0;
  if (k <= 0 || k % 8 != 0 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) ||
      ((uintptr_t)q_out & 15) || ((uintptr_t)pages & 15) || ((uintptr_t)angles & 15))
    return (int)cudaErrorInvalidValue;
  if ((head_dim != 64 && head_dim != 128) || n % head_dim || q_col % head_dim || k_col % head_dim || v_col % head_dim ||
      nq < 0 || nkv < 0 || (nkv > 0 && (slots == nullptr || pages == nullptr || page_size < 1)))
    return (int)cudaErrorInvalidValue;
  const QkvParts parts = {head_dim, q_col, k_col, v_col, nq, nkv, eps, (const float2*)angles, slots, (bf16*)q_out,
                          (bf16*)pages, page_size, num_slots};
  return launch_width<EPI_QKV, 256>(a, w, out, m, n, k, 0, 1.f, 0.f, parts, err, stream);
}
