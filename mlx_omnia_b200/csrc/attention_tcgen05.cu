// Paged causal prefill attention in bfloat16 on the 5th-generation tensor cores, compiled for
// one head size and one group size:
//   -DHEAD_DIM=64|128   -DGROUP=g (query heads per key/value head, g <= 16)
//
// A block owns up to 128 rows, each row a (token, query head of the group) pair of ONE
// key/value head and one request, and walks the visible keys in tiles of 64 (two blocks share an SM,
// so one block's softmax overlaps the other's matrix products):
//   S = Q K^T   tcgen05.mma (M 128, N 64) over the head size, accumulator in tensor memory
//   softmax     four warps, one thread per row: tcgen05.ld the scores, mask, running maximum and
//               sum in float32, exp2, P rounded to bfloat16 and stored (tcgen05.st) over the scores
//               it came from: the score accumulator is double-buffered, so P of one tile and S of
//               the next never share columns, and a tile's softmax need not wait for the product
//               of the tile before
//   O += P V    tcgen05.mma (M 128, N head size) over the tile's keys, P read from tensor memory,
//               accumulator in tensor memory. The exponent's offset follows a row's maximum lazily:
//               it moves (and the accumulator is rescaled in tensor memory, after the products so
//               far) only when the maximum has grown by more than 2^8 since, which after the first
//               tiles is rare; until then P simply exceeds 1, which float32 sums do not mind
// Warps 0 (K) and 6 (V) feed the rings of K and V stages with TMA, one box of 16 keys x 64 dims per page
// group (the block table is read there; page sizes must be multiples of 16); warps 1 and 7 issue the
// two kinds of MMA; warps 2-5 are the softmax and the epilogue (normalise, optional sigmoid gate, store). The score
// accumulator is double-buffered, so S of the next tile is computed while this tile's softmax runs.
// Key groups whose page is not loaded (beyond the request, or given back behind a window) are
// masked in S and skipped in P V, so stale shared memory never reaches the arithmetic; the rows
// of the last loaded group that lie past the block's last key (the unwritten tail of the
// request's last page) are cleared in the V tile, so whatever a page's previous owner left
// there (a NaN included) meets its zero weight as a zero.
//
// A block that would walk many tiles (a portion of a prompt over a long context; the last blocks of a
// long prompt) can be listed as several PARTS, each a run of the block's key tiles: a part leaves its
// unnormalised accumulator, its exponent offset and its sum in a workspace (float32, laid out so that
// a warp's accesses are whole lines), draws a ticket, and the part that draws the last one adds the
// parts in their order (the result does not depend on which part came last), normalises, applies
// the gate and stores. Nobody waits for another block.
//
// Every wait on a barrier is bounded: when the bound is hit the block raises OMNIA_ERR_TIMEOUT
// in the error word, every role leaves its loop, the producer waits (bounded) for loads in
// flight, the block frees its tensor memory and returns.
#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
#ifndef GROUP
#define GROUP 2
#endif

#include "attention_tcgen05.cuh"

namespace {

constexpr int D = HEAD_DIM;
static_assert(D == 64 || D == 128, "the tcgen05 attention kernel takes head sizes 64 and 128");
static_assert(GROUP >= 1 && GROUP <= 16, "group size must be 1..16");
constexpr int DH = D / 64;                 // 64-wide halves of a head
constexpr int BM = 128, BN = 64;      // rows per block, keys per tile
constexpr int TOKENS = BM / GROUP;         // tokens per block
constexpr int ROWS = TOKENS * GROUP;       // rows in use (<= 128)
constexpr int K_STAGES = 2, V_STAGES = 3;
static_assert(K_STAGES == 2, "a K stage is freed by the score buffer of the same index");  // ring depths (a K stage is free once its scores are computed, a V stage
                                           // only after its product, two tiles later: V needs the deeper ring)
constexpr int THREADS = 256;  // warps: 0 K producer, 1 issuer of Q K^T, 2-5 softmax, 6 V producer, 7 issuer of P V
constexpr uint32_t HALF_BYTES = 128 * 128;           // 128 rows of 128 bytes
constexpr uint32_t Q_BYTES = DH * HALF_BYTES;
constexpr uint32_t TILE_HALF = BN * 128;             // 64 keys of 128 bytes
constexpr uint32_t K_BYTES = DH * TILE_HALF, V_BYTES = DH * TILE_HALF;
constexpr uint32_t GROUP_BYTES = 16 * 128;           // one TMA box: 16 keys x 64 dims
constexpr uint32_t TMEM_COLS = 256;                  // two blocks share an SM's 512 columns
constexpr uint32_t S_COL = 0, O_COL = 128;

// The four softmax warps among themselves.
__device__ __forceinline__ void softmax_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

}  // namespace

// grid (blocks of the work list); THREADS threads. work[b] = (request, first token of the block among
// the request's tokens of this step, key/value head, first key tile of this part counted from the
// block's first, tiles of this part (< 0: all the block's), parts of the block + 256 x this part's
// number, place of the block's first part in the workspace, number of the block among the split
// ones); request < 0: nothing to do. The caller lists the longest first.
constexpr int WORK_INTS = 8;
constexpr int MAX_PARTS = 16;
constexpr int PART_FLOATS = BM * D + 2 * BM;  // a part in the workspace: O as [D / 4][128 rows] float4, then offsets, then sums
__global__ void __launch_bounds__(THREADS, 2)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                                 const __grid_constant__ CUtensorMap map_gate, int gate_tma,
                                 const int* __restrict__ block_table, const int* __restrict__ cu_seqlens,
                                 const int* __restrict__ seq_lens, const int* __restrict__ work,
                                 const bf16* __restrict__ gate, int gate_stride, bf16* __restrict__ out,
                                 float* __restrict__ partial, int* __restrict__ tickets,
                                 int max_pages, int num_pages, int nq, int nkv, int page_size, int window,
                                 float scale, int* err) {
  if (work[WORK_INTS * blockIdx.x] < 0) return;  // a place of the list that this step does not use
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // The swizzled tiles need a base on 1024 bytes; the dynamic area starts on one (nothing static
  // precedes it). Two blocks per SM leave no room for padding, so this is checked, not forced.
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0) atomicOr(err, OMNIA_ERR_TIMEOUT);
    return;
  }
  unsigned char* q_s = smem_raw;
  unsigned char* k_s = q_s + Q_BYTES;            // K_STAGES tiles of keys
  unsigned char* v_s = k_s + K_STAGES * K_BYTES;  // V_STAGES tiles of values
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + V_STAGES * V_BYTES);
  // bars: q_full | k_full[2] | v_full[3] | v_done[3] | s_full[2] | p_full[2] | g_full
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile uint32_t* group_mask = reinterpret_cast<volatile uint32_t*>(tmem_holder + 2);  // [V_STAGES]
  volatile int* drawn = reinterpret_cast<volatile int*>(tmem_holder + 2 + V_STAGES);  // the ticket this part drew

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* item = work + WORK_INTS * blockIdx.x;
  const int seq = item[0], tok0 = item[1], kvh = item[2], parts = item[5] & 255, part = item[5] >> 8, slot0 = item[6],
            unit = item[7];
  const int q_begin = cu_seqlens[seq], q_len = cu_seqlens[seq + 1] - q_begin;
  const int pos0 = seq_lens[seq] - q_len + tok0;      // position of the block's first token
  const int tokens = min(TOKENS, q_len - tok0);
  const int rows = tokens * GROUP;
  const int last = pos0 + tokens - 1;                                   // last key any row sees
  const int first = window > 0 ? max(0, pos0 - window + 1) : 0;         // first key any row sees
  const int last_tile = last / BN;
  const int tile0 = first / BN + (item[4] < 0 ? 0 : item[3]);
  const int n_tiles = item[4] < 0 ? last_tile - tile0 + 1 : item[4];
  const bool whole = parts <= 1;  // this block does all of its rows' keys and stores the result itself

  const uint32_t bar0 = smem_u32(bars);
  const uint32_t q_full = bar0, k_full0 = bar0 + 8, v_full0 = k_full0 + 8 * K_STAGES, v_done0 = v_full0 + 8 * V_STAGES,
                 s_full0 = v_done0 + 8 * V_STAGES, p_full0 = s_full0 + 16, g_full = p_full0 + 16;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < K_STAGES; ++s) mbar_init(k_full0 + 8 * s, 1);
    for (int s = 0; s < V_STAGES; ++s) mbar_init(v_full0 + 8 * s, 1), mbar_init(v_done0 + 8 * s, 1);
    for (int s = 0; s < 2; ++s) mbar_init(s_full0 + 8 * s, 1), mbar_init(p_full0 + 8 * s, 128);  // one per score buffer
    mbar_init(g_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;
  // Everything so far needed nothing from the kernel before this one and ran while it finished
  // (the launch is a programmatic dependent launch); from here on its results are read.
  OMNIA_TRACE_BLOCK(2);
  pdl_wait();
  pdl_launch_dependents();
  OMNIA_TRACE_BLOCK(3);

  if (warp == 0 || warp == 6) {
    // ---- producers: warp 0 loads Q once, then the K tiles; warp 6 the V tiles. Issuing a box keeps
    // a warp busy for about 70 ns: one warp for both rings spent more than half a tile's time on it
    // (2,048 tokens: 61 us with one warp, 52 us with one per ring; two per ring: no faster). ------
    const int which = warp == 0 ? 0 : 1;  // 0 keys, 1 values
    if (warp == 0 && lane == 0) {
      mbar_expect_tx(q_full, DH * ROWS * 128);
      for (int h = 0; h < DH; ++h)
        tma_load_3d(smem_u32(q_s) + h * HALF_BYTES, &map_q, q_full, h * 64, kvh * GROUP, q_begin + tok0);
    }
    // Lane = group * DH + half: each of the tile's boxes (16 keys x 64 dims) is issued by its own lane.
    const int* table = block_table + (size_t)seq * max_pages;
    if (lane == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
    const int g = lane / DH, h = lane % DH;
    const bool active = lane < (BN / 16) * DH;
    // The page of this lane's group in tile t (-2: the group lies outside what the block reads).
    // Page numbers are fetched a whole tile before they are used, so the table's latency is hidden.
    auto lookup = [&](int t) {
      const int pos = (tile0 + t) * BN + g * 16;
      return (active && t < n_tiles && pos <= last && pos + 15 >= first) ? table[pos / page_size] : -2;
    };
    bool ok = true;
    int issued = 0;
    auto load_tile = [&](int j, int page) {
      // A K stage is free when the scores computed from it are there (s_full of the same index: there
      // are as many score buffers as K stages), a V stage when its product is done (v_done).
      const int stages = which ? V_STAGES : K_STAGES, s = j % stages;
      const uint32_t full = (which ? v_full0 : k_full0) + 8 * s, empty = (which ? v_done0 : s_full0) + 8 * s;
      if (lane == 0 && j >= stages) ok = mbar_wait(empty, ((j / stages) & 1) ^ 1, abort_flag);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return;
      if (lane == 0) STAMP(0, j, which * 2);
      const int pos = (tile0 + j) * BN + g * 16;
      bool load = page != -2;
      if (load && (page < 0 || page >= num_pages)) {
        // A page behind the window may have been given back; one the block really reads may not.
        if (pos >= first) atomicOr(err, OMNIA_ERR_PAGE);
        load = false;
      }
      const uint32_t loaded = __ballot_sync(0xffffffffu, load);
      if (lane == 0) {
        if (which) {
          uint32_t mask = 0;
#pragma unroll
          for (int x = 0; x < BN / 16; ++x) mask |= ((loaded >> (x * DH)) & 1u) << x;
          group_mask[s] = mask;
        }
        mbar_expect_tx(full, __popc(loaded) * GROUP_BYTES);
      }
      __syncwarp();
      if (load) {
        const int y = (((page * 2 + which) * nkv + kvh) * page_size) + pos % page_size;
        const uint32_t dst = smem_u32(which ? v_s + s * V_BYTES : k_s + s * K_BYTES) + h * TILE_HALF + g * GROUP_BYTES;
        tma_load_2d(dst, &map_kv, full, h * 64, y);
      }
      if (lane == 0) STAMP(0, j, which * 2 + 1);
      issued = j + 1;
    };
    // A K slot is free again as soon as its scores are computed, a V slot when its P V is: each
    // ring runs up to two tiles ahead of the tensor core.
    int page_cur = lookup(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int page_next = lookup(j + 1);
      load_tile(j, page_cur);
      page_cur = page_next;
    }
    if (lane == 0 && *abort_flag) {
      const uint32_t full0 = which ? v_full0 : k_full0;
      const int stages = which ? V_STAGES : K_STAGES;
      for (int j = max(0, issued - stages); j < issued; ++j)
        for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(full0 + 8 * (j % stages), (j / stages) & 1); ++i) {
        }
      for (uint32_t i = 0; warp == 0 && i < WAIT_LIMIT && !mbar_try(q_full, 0); ++i) {
      }
    }
  } else if (warp == 1) {
    // ---- issuer of the score products: S[j & 1] = Q K_j^T --------------------------------------------
    // The two kinds of product are issued by two threads (this warp and warp 7). The products of one
    // accumulator depend on one another and run one at a time, some 50 to 100 ns each whatever their
    // size; a single thread issuing a tile's twelve kept at most one chain in flight and a tile took
    // 1.27 us, two threads keep the scores' chain and the values' chain going side by side (1.06 us).
    // What one thread's products must wait for of the other's goes through barriers: a score buffer
    // is written again only when the P V product that read P from it is done (v_done, two tiles back).
    if (lane == 0) {
      constexpr uint32_t instr_s = idesc(BM, BN, false);
      // Descriptors differ only in their address field (the low 14 bits, in units of 16 bytes).
      const uint64_t q_desc = desc_k_major(smem_u32(q_s));
      uint64_t k_desc[K_STAGES];
      for (int s = 0; s < K_STAGES; ++s) k_desc[s] = desc_k_major(smem_u32(k_s + s * K_BYTES));
      bool ok = mbar_wait(q_full, 0, abort_flag);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % K_STAGES;
        ok = mbar_wait(k_full0 + 8 * s, (j / K_STAGES) & 1, abort_flag);
        if (ok && j >= 2) ok = mbar_wait(v_done0 + 8 * ((j - 2) % V_STAGES), ((j - 2) / V_STAGES) & 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        STAMP(1, j, 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma(tmem_base + S_COL + (j & 1) * BN, q_desc + (((kk / 4) * HALF_BYTES + (kk % 4) * 32) >> 4),
               k_desc[s] + (((kk / 4) * TILE_HALF + (kk % 4) * 32) >> 4), instr_s, kk != 0);
        umma_commit(s_full0 + 8 * (j & 1));  // the scores are there, and with them the K stage is free again
        STAMP(1, j, 3);
      }
    }
  } else if (warp == 7) {
    // ---- issuer of the value products: O += P_j V_j ---------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t instr_o = idesc(BM, D, true);
      uint64_t v_desc[V_STAGES];
      for (int s = 0; s < V_STAGES; ++s) v_desc[s] = desc_mn_major(smem_u32(v_s + s * V_BYTES), TILE_HALF);
      uint32_t accumulate = 0;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % V_STAGES;
        ok = mbar_wait(v_full0 + 8 * s, (j / V_STAGES) & 1, abort_flag) &&
             mbar_wait(p_full0 + 8 * (j & 1), (j >> 1) & 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        STAMP(1, j, 1);
        const uint32_t mask = group_mask[s];
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          if (!(mask & (1u << kk))) continue;  // keys never loaded: their P is zero, their V is stale
          // P: 16 keys are eight columns of packed bfloat16 pairs in the score buffer's place
          umma_ts(tmem_base + O_COL, tmem_base + S_COL + (j & 1) * BN + kk * 8, v_desc[s] + ((kk * GROUP_BYTES) >> 4),
                  instr_o, accumulate);
          accumulate = 1;
        }
        umma_commit(v_done0 + 8 * s);  // the product is done: the V stage is free, and O may be read or rescaled
        STAMP(1, j, 2);
      }
    }
  } else {
    // ---- softmax and epilogue: one thread per row ---------------------------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const bool live = row < rows;
    // A row past the block's last token (a prompt's last block need not be full) sees what the last
    // token sees: it is never stored, and with a range of its own (none) its warp would take the
    // masked path through every tile, which set the pace of a prompt's longest block (3,000 tokens:
    // 85 us a layer against 63 for 3,008).
    const int pos = min(pos0 + row / GROUP, last);
    const int row_hi = pos;
    const int row_lo = window > 0 ? max(0, pos - window + 1) : 0;
    const uint32_t lane_field = (uint32_t)(quarter * 32) << 16;
    const float sl2 = scale * LOG2E;
    float m = -INFINITY, l = 0.f;
    bool ok = true, gate_issued = false;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int key0 = (tile0 + j) * BN;
      ok = mbar_wait(s_full0 + 8 * (j & 1), (j >> 1) & 1, abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (whole && j == n_tiles - 1 && row == 0 && gate_tma) {
        // The last scores are there, so Q has been read for the last time: the block's gate
        // values (the same rows and columns as Q, of another matrix) take its place, on their
        // way while the last softmax and product run.
        mbar_expect_tx(g_full, DH * ROWS * 128);
        for (int h = 0; h < DH; ++h)
          tma_load_3d(smem_u32(q_s) + h * HALF_BYTES, &map_gate, g_full, h * 64, kvh * GROUP, q_begin + tok0);
        gate_issued = true;
      }
      OMNIA_TRACE_IF(row == 0 && j == 0, 5);
      if (row == 0) STAMP(2, j, 0);
      const uint32_t s_addr = tmem_base + lane_field + S_COL + (j & 1) * BN;
      // Which keys of the tile this row sees; a tile that the whole warp sees whole needs no masks.
      const int lo = max(row_lo - key0, 0), hi = min(row_hi - key0, BN - 1);  // visible columns [lo, hi]
      const bool unmasked = __all_sync(0xffffffffu, lo == 0 && hi == BN - 1);
      // The row's 64 scores, read once; then their maximum.
      static_assert(BN == 64, "the softmax below handles one 64-column pass per tile");
      uint32_t v[64];
      tmem_load32(s_addr, v);
      tmem_load32(s_addr + 32, v + 32);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      float tile_max = -INFINITY;
      if (unmasked) {
        float part[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains instead of one of 64
#pragma unroll
        for (int i = 0; i < 64; ++i) part[i & 3] = fmaxf(part[i & 3], __uint_as_float(v[i]));
        tile_max = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i >= lo && i <= hi) tile_max = fmaxf(tile_max, __uint_as_float(v[i]));
      }
      if (row == 0) STAMP(2, j, 1);
      // The offset of the exponent (m) follows the row's maximum lazily: a softmax does not care
      // which offset it is computed with, so m moves only when the maximum has outgrown it by more
      // than 2^RESCALE_STEP (P then stays below that), and only then is the accumulator rescaled.
      float alpha = 1.f;
      if (tile_max > m) {
        if (m == -INFINITY) {
          m = tile_max;  // the row's first keys: nothing has been accumulated yet
        } else if ((tile_max - m) * sl2 > RESCALE_STEP) {
          alpha = fast_exp2((m - tile_max) * sl2);
          m = tile_max;
        }
      }
      const float offset = m == -INFINITY ? 0.f : m * sl2;
      // P = exp2(s * scale * log2e - offset), rounded to bfloat16.
      float sums[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[32];
      if (unmasked) {
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), sl2, -offset));
          const float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), sl2, -offset));
          sums[(i >> 1) & 3] += p0 + p1;
          packed[i / 2] = pack_bf16(p0, p1);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          float p[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = i + e;
            p[e] = (col >= lo && col <= hi) ? fast_exp2(fmaf(__uint_as_float(v[i + e]), sl2, -offset)) : 0.f;
          }
          sums[(i >> 1) & 3] += p[0] + p[1];
          packed[i / 2] = pack_bf16(p[0], p[1]);
        }
      }
      const float sum = (sums[0] + sums[1]) + (sums[2] + sums[3]);
      if (__any_sync(0xffffffffu, alpha != 1.f)) {
        // The products so far must be done before the accumulator is rescaled.
        if (j > 0) {
          ok = mbar_wait(v_done0 + 8 * ((j - 1) % V_STAGES), ((j - 1) / V_STAGES) & 1, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_load32(tmem_base + lane_field + O_COL + c, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_store32(tmem_base + lane_field + O_COL + c, o);
        }
      }
      if (row == 0) STAMP(2, j, 2);
      l *= alpha;
      // P takes the place of the scores it came from (this buffer's next scores are two tiles away,
      // and their product is issued after this tile's P V): 64 keys are 32 columns of packed pairs.
      tmem_store32(s_addr, packed);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      l += sum;
      if (tile0 + j == last_tile && ((last + 1) & 15)) {
        // The last group of 16 keys reaches past the block's last key. Those rows of V get a
        // zero weight, but what they hold need not be a number: past the request's last token
        // the page still holds whatever its previous owner left (0 x NaN is NaN). Clear them in
        // the tile once it has landed; the fence orders the stores before the P V product.
        const int s = j % V_STAGES;
        ok = mbar_wait(v_full0 + 8 * s, (j / V_STAGES) & 1, abort_flag);
        if (!ok) break;
        const int r0 = last - key0 + 1, r1 = (r0 + 15) & ~15;  // rows [r0, r1) of the tile
        unsigned char* v_tile = v_s + s * V_BYTES;
        for (int i = row; i < (r1 - r0) * DH * 8; i += 128) {
          const int piece = i & 7, h = (i >> 3) % DH, r = r0 + (i >> 3) / DH;
          *reinterpret_cast<uint4*>(v_tile + h * TILE_HALF + r * 128 + piece * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // V is read by the tensor core (async proxy)
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(p_full0 + 8 * (j & 1));
      if (row == 0) STAMP(2, j, 3);
      if (lane == 0) STAMP(3, j, quarter);
    }
    // Epilogue: O / l, gate, store. A thread owns a row, so a warp's loads and stores go to 32
    // different rows, each a trip to L2 of its own: read that way (two bytes at a time, then
    // sixteen) the gate cost a block 30 and 13 us. It comes by TMA into Q's place instead (see the
    // loop) and is read from shared memory, 16 bytes at a time, like everything stored.
    OMNIA_TRACE_IF(row == 0, 6);
    const size_t token = (size_t)(q_begin + tok0 + row / GROUP);
    const int head = kvh * GROUP + row % GROUP;
    const bf16* gp = gate ? gate + token * gate_stride + (size_t)head * D : nullptr;
    const bool gate_wide = gp != nullptr && (reinterpret_cast<uintptr_t>(gp) & 15) == 0;
    if (ok) ok = mbar_wait(v_done0 + 8 * ((n_tiles - 1) % V_STAGES), ((n_tiles - 1) / V_STAGES) & 1, abort_flag);
    if (ok && whole && gate_tma) ok = mbar_wait(g_full, 0, abort_flag);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    OMNIA_TRACE_IF(row == 0, 7);
    if (!whole) {
      // ---- a part: leave O, the exponent's offset and the sum in the workspace, draw a ticket. The
      // four warps stay together through the named barriers whatever `ok` says. -----------------------
      float* mine = partial + (size_t)(slot0 + part) * PART_FLOATS;
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_load32(tmem_base + lane_field + O_COL + c, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            __stcg(reinterpret_cast<float4*>(mine) + (size_t)((c + i) / 4) * BM + row,
                   make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]), __uint_as_float(o[i + 2]),
                               __uint_as_float(o[i + 3])));
        }
        __stcg(mine + BM * D + row, m == -INFINITY ? -INFINITY : m * sl2);
        __stcg(mine + BM * D + BM + row, l);
      }
      __threadfence();
      softmax_sync();
      if (row == 0) *drawn = *abort_flag ? -1 : atomicAdd(tickets + unit, 1);
      softmax_sync();
      if (*drawn == parts - 1) {
        // ---- the last part to arrive: every row's weights of the parts (the exponent offsets brought
        // to their largest) and the reciprocal of its sum go to shared memory, in the K ring's place;
        // all eight warps then add the parts (below, behind the block's barrier) ---------------------
        __threadfence();
        if (row == 0) tickets[unit] = 0;  // for the next launch
        if (row == 0 && gate_tma) {
          // Q has been read for the last time: the gate values of the block's rows take its place.
          mbar_expect_tx(g_full, DH * ROWS * 128);
          for (int h = 0; h < DH; ++h)
            tma_load_3d(smem_u32(q_s) + h * HALF_BYTES, &map_gate, g_full, h * 64, kvh * GROUP, q_begin + tok0);
        }
        const float* all = partial + (size_t)slot0 * PART_FLOATS;
        float* weights = reinterpret_cast<float*>(k_s);  // [parts + 1][128]: the parts' weights, then 1 / sum
        float top = -INFINITY, total = 0.f;
        for (int q = 0; q < parts; ++q) top = fmaxf(top, __ldcg(all + (size_t)q * PART_FLOATS + BM * D + row));
        for (int q = 0; q < parts; ++q) {
          const float offset = __ldcg(all + (size_t)q * PART_FLOATS + BM * D + row);
          const float w = offset != -INFINITY ? fast_exp2(offset - top) : 0.f;
          weights[q * BM + row] = w;
          total += w * __ldcg(all + (size_t)q * PART_FLOATS + BM * D + BM + row);
        }
        weights[parts * BM + row] = total > 0.f ? 1.f / total : 0.f;
      }
    }
    if (ok && whole) {
      // 64 dims of the row's accumulator in one go (two loads side by side; eight dims a turn with the
      // next turn's columns on their way took longer: every turn waited for a load), then eight dims
      // at a time: normalise, gate, 16 bytes stored.
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = out + (token * nq + head) * D;
      const uint32_t o_addr = tmem_base + lane_field + O_COL;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 64) {
        uint32_t acc[64];
        tmem_load32(o_addr + c0, acc);
        tmem_load32(o_addr + c0 + 32, acc + 32);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (!live) continue;
#pragma unroll
        for (int i = 0; i < 64; i += 8) {
          const int c = c0 + i;
          uint4 g = make_uint4(0u, 0u, 0u, 0u);
          if (gate_tma) {
            // Row `row` of the 64-dim half c / 64, 128 bytes a row, its 16-byte pieces swizzled by the row.
            g = *reinterpret_cast<const uint4*>(q_s + (c / 64) * HALF_BYTES + row * 128 + ((((c % 64) / 8) ^ (row & 7)) << 4));
          } else if (gate_wide) {
            g = __ldg(reinterpret_cast<const uint4*>(gp + c));
          } else if (gp) {
            g.x = pack_bf16(__bfloat162float(gp[c]), __bfloat162float(gp[c + 1]));
            g.y = pack_bf16(__bfloat162float(gp[c + 2]), __bfloat162float(gp[c + 3]));
            g.z = pack_bf16(__bfloat162float(gp[c + 4]), __bfloat162float(gp[c + 5]));
            g.w = pack_bf16(__bfloat162float(gp[c + 6]), __bfloat162float(gp[c + 7]));
          }
          const uint32_t g2[4] = {g.x, g.y, g.z, g.w};
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float a = __uint_as_float(acc[i + 2 * e]) * inv, b2 = __uint_as_float(acc[i + 2 * e + 1]) * inv;
            if (gp) {
              const float2 gate2 = sigmoid_pair(g2[e]);
              a *= gate2.x;
              b2 *= gate2.y;
            }
            w[e] = pack_bf16(a, b2);
          }
          *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    } else if (whole && gate_issued) {
      // Giving up: the gate's copy must land before the block's shared memory goes away.
      for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(g_full, 0); ++i) {
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (!whole && *drawn == parts - 1) {
    // ---- the merge, by all eight warps: an item is eight dims of a row, neighbouring threads take
    // neighbouring rows (whole lines of the workspace), the parts are added in their order ------------
    static_assert((MAX_PARTS + 1) * BM * sizeof(float) <= K_STAGES * K_BYTES, "the parts' weights fit the K ring's place");
    bool merged = true;
    if (gate_tma) {
      merged = mbar_wait(g_full, 0, abort_flag);
      // Giving up: the gate's copy must still land before the block's shared memory goes away.
      for (uint32_t i = 0; !merged && i < WAIT_LIMIT && !mbar_try(g_full, 0); ++i) {
      }
    }
    const float* all = partial + (size_t)slot0 * PART_FLOATS;
    const float* weights = reinterpret_cast<const float*>(k_s);
    if (merged) {
#pragma unroll 2
      for (int item = threadIdx.x; item < BM * (D / 8); item += THREADS) {
        const int row = item % BM, c = (item / BM) * 8;
        if (row >= rows) continue;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int q = 0; q < parts; ++q) {
          const float4* src = reinterpret_cast<const float4*>(all + (size_t)q * PART_FLOATS) + (size_t)(c / 4) * BM + row;
          const float4 a = __ldcg(src), b2 = __ldcg(src + BM);
          const float w = weights[q * BM + row];
          acc[0] += w * a.x, acc[1] += w * a.y, acc[2] += w * a.z, acc[3] += w * a.w;
          acc[4] += w * b2.x, acc[5] += w * b2.y, acc[6] += w * b2.z, acc[7] += w * b2.w;
        }
        const float inv = weights[parts * BM + row];
        const size_t token = (size_t)(q_begin + tok0 + row / GROUP);
        const int head = kvh * GROUP + row % GROUP;
        uint4 g = make_uint4(0u, 0u, 0u, 0u);
        if (gate_tma) {
          g = *reinterpret_cast<const uint4*>(q_s + (c / 64) * HALF_BYTES + row * 128 + ((((c % 64) / 8) ^ (row & 7)) << 4));
        } else if (gate != nullptr) {
          const bf16* gp = gate + token * gate_stride + (size_t)head * D + c;
          g.x = pack_bf16(__bfloat162float(gp[0]), __bfloat162float(gp[1]));
          g.y = pack_bf16(__bfloat162float(gp[2]), __bfloat162float(gp[3]));
          g.z = pack_bf16(__bfloat162float(gp[4]), __bfloat162float(gp[5]));
          g.w = pack_bf16(__bfloat162float(gp[6]), __bfloat162float(gp[7]));
        }
        const uint32_t g2[4] = {g.x, g.y, g.z, g.w};
        uint32_t w4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float a = acc[2 * e] * inv, b2 = acc[2 * e + 1] * inv;
          if (gate != nullptr) {
            const float2 gate2 = sigmoid_pair(g2[e]);
            a *= gate2.x;
            b2 *= gate2.y;
          }
          w4[e] = pack_bf16(a, b2);
        }
        *reinterpret_cast<uint4*>(out + (token * nq + head) * D + c) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
      }
    }
  }
  OMNIA_TRACE_BLOCK(4);
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(err, OMNIA_ERR_TIMEOUT);
}

// ---- host side -------------------------------------------------------------------------------

#ifdef ATTN_TIMING
extern "C" int omnia_attention_timing(unsigned long long* host, int count) {
  return (int)cudaMemcpyFromSymbol(host, g_timing, sizeof(unsigned long long) * count);
}
#endif

extern "C" int omnia_attention_tcgen05_part_floats(void) { return PART_FLOATS; }

extern "C" int omnia_attention_tcgen05_info(int* head_dim, int* group, int* tokens_per_block) {
  *head_dim = HEAD_DIM;
  *group = GROUP;
  *tokens_per_block = TOKENS;
  return 0;
}

// q: [tokens, nq, D]; pages: [num_pages, 2, nkv, page_size, D]; page_size a multiple of 16.
// work: `blocks` items of 8 ints (see the kernel). partial: float32 workspace, omnia_attention_tcgen05_part_floats()
// floats for every part of a split block (null when no block is split); tickets: one int per split
// block, zero before the first launch (the kernel leaves them zero).
extern "C" int omnia_attention_prefill_tcgen05(const void* q, int tokens, const void* pages, const int* block_table,
                                               const int* cu_seqlens, const int* seq_lens, const int* work,
                                               int blocks, const void* gate, int gate_stride, void* out,
                                               float* partial, int* tickets,
                                               int max_pages, int num_pages, int nq, int nkv, int page_size,
                                               int window, float scale, int* err, cudaStream_t stream) {
  if (blocks == 0) return 0;
  if (nq != nkv * GROUP || page_size % 16 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)pages & 15))
    return (int)cudaErrorInvalidValue;
  CUtensorMap map_q, map_kv, map_gate;
  int gate_tma = 0;
  const int made = attention_maps(&map_q, &map_kv, &map_gate, &gate_tma, q, tokens, pages, gate, gate_stride, num_pages, nq,
                                  nkv, page_size, D, GROUP, TOKENS);
  if (made != 0) return made;
  constexpr size_t smem = Q_BYTES + K_STAGES * K_BYTES + V_STAGES * V_BYTES + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  launch_pdl(attention_prefill_tcgen05_kernel, blocks, THREADS, smem, stream,
             map_q, map_kv, map_gate, gate_tma, block_table, cu_seqlens, seq_lens, work, (const bf16*)gate, gate_stride, (bf16*)out,
             partial, tickets, max_pages, num_pages, nq, nkv, page_size, window, scale, err);
  return OMNIA_LAUNCH_RESULT();
}
