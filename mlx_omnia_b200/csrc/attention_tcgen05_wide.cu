// Paged causal prefill attention in bfloat16 on the 5th-generation tensor cores, one block to an SM,
// for steps whose blocks are few and long (a whole prompt of some hundred to some thousand tokens);
// attention_tcgen05.cu, two blocks to an SM, takes the others. Compiled for one head size and one
// group size:
//   -DHEAD_DIM=64|128   -DGROUP=g (query heads per key/value head, g <= 16)
//
// A block owns up to 128 rows, each row a (token, query head of the group) pair of ONE key/value
// head and one request, has all of its SM's tensor memory (three score buffers of 128 columns and
// the accumulator) and walks the visible keys in score tiles of 128:
//   S = Q K^T   tcgen05.mma (M 128, N 128) over the head size. A product with its 128-row operand in
//               shared memory occupies the tensor core for 65 to 80 ns however few columns it has, so
//               a tile of 128 keys costs the eight products that a tile of 64 would
//   softmax     two teams of four warps, a thread per row in each, take turns with the tiles: one
//               team's exponentials run while the other reads its scores and finds its maximum. What
//               a tile needs of the tile before, the exponent's offset, goes through shared memory
//               behind a pair of named barriers. Two passes over the scores, 32 at a time (first the
//               maximum, then P), keep a thread's registers few; the pairs of 16 keys (P rounded to
//               bfloat16) take the place of the first eight of those keys' scores
//   O += P V    tcgen05.mma (M 128, N head size), P read from tensor memory, V in stages of 64 keys.
//               The exponent's offset follows a row's maximum lazily, as in the other kernel
// Warps 0, 1 feed the ring of K tiles and warps 12, 13 the ring of V stages with TMA, a box of 16 keys
// x 64 dims per page group (issuing a box keeps a warp busy for some 70 ns whatever its size, so each
// ring has two warps that take turns); warps 2 and 3 issue the two kinds of product; warps 4-11 are
// the softmax and the epilogue (each team normalises, gates and stores half of the dims). Masking of
// groups that are not loaded, the cleared tail of the last V stage and the bounded waits are the other
// kernel's; the work list is the same (tiles counted in 64 keys), but every block does all of its keys:
// a list that cuts a block into parts is refused. The named barriers cannot be bounded, so every softmax warp passes them
// once a tile whatever has gone wrong, and `ok` is kept the same within a warp.
//
// Measured on a B200 (16/8 heads of 128, with the gate), against the two-blocks-to-an-SM kernel: a
// whole prompt of 1,024 / 2,048 / 3,000 tokens 19 / 37 / 66 us against 24 / 44 / 85; of 4,096 / 8,192
// tokens 101 / 323 against 88 / 290 (a block's 7 us of start and epilogue overlap nothing here, and in
// the steady state both kernels take 1.35 us for 128 keys); portions cut into parts 75 against 57
// (512 tokens over 8,192).
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
constexpr int BM = 128;                    // rows per block
constexpr int SN = 128;                    // keys per score tile
constexpr int BN = 64;                     // keys per V stage, which is also the unit of the work list
constexpr int HALVES = SN / BN;            // V stages per score tile
constexpr int TOKENS = BM / GROUP;         // tokens per block
constexpr int ROWS = TOKENS * GROUP;       // rows in use (<= 128)
// Ring depths: a K stage is freed by the score buffer of the same index (its scores are computed), a
// V stage only after its product. With two score buffers the chain of a tile's softmax, its P V and
// the scores two tiles on set the pace (8,192 tokens: 350 us; with three: 333).
constexpr int S_BUFS = 3, K_STAGES = S_BUFS, V_STAGES = 4;
// Warps: 0, 1 fill the K stages in turns; 2 issues Q K^T (and owns the tensor memory); 3 issues P V;
// 4-7 and 8-11 are the softmax teams (a warp reads the tensor-memory lanes of its number modulo
// four); 12, 13 fill the V stages in turns.
constexpr int FEEDERS = 2;  // warps per ring
constexpr int THREADS = 32 * 14;
constexpr int WARP_K = 0, WARP_QK = 2, WARP_PV = 3, WARP_SOFTMAX = 4, WARP_V = 12;
constexpr int SOFTMAX_THREADS = 256;  // two teams, a thread per row in each
constexpr uint32_t HALF_BYTES = 128 * 128;           // 128 rows of 128 bytes
constexpr uint32_t Q_BYTES = DH * HALF_BYTES;
constexpr uint32_t TILE_HALF = BN * 128;             // a V stage's 64 keys of 128 bytes
constexpr uint32_t K_TILE_HALF = SN * 128;           // a K stage's keys of 128 bytes
constexpr uint32_t K_BYTES = DH * K_TILE_HALF, V_BYTES = DH * TILE_HALF;
constexpr uint32_t GROUP_BYTES = 16 * 128;           // one TMA box: 16 keys x 64 dims
constexpr uint32_t TMEM_COLS = 512;                  // the score buffers and the accumulator: all of the SM's columns
constexpr uint32_t S_COL = 0, O_COL = S_BUFS * SN;

// The softmax warps among themselves.
__device__ __forceinline__ void softmax_sync() { asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_THREADS) : "memory"); }

}  // namespace

// grid (blocks of the work list); THREADS threads. work[b] = (request, first token of the block among
// the request's tokens of this step, key/value head, 0, -1, 1, 0, 0): the other kernel's items, of
// which only whole blocks are taken; request < 0: nothing to do. The caller lists the longest first.
constexpr int WORK_INTS = 8;
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                                 const __grid_constant__ CUtensorMap map_gate, int gate_tma,
                                 const int* __restrict__ block_table, const int* __restrict__ cu_seqlens,
                                 const int* __restrict__ seq_lens, const int* __restrict__ work,
                                 const bf16* __restrict__ gate, int gate_stride, bf16* __restrict__ out,
                                 int max_pages, int num_pages, int nq, int nkv, int page_size, int window,
                                 float scale, int* err) {
  if (work[WORK_INTS * blockIdx.x] < 0) return;  // a place of the list that this step does not use
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // The swizzled tiles need a base on 1024 bytes; the dynamic area starts on one (nothing static
  // precedes it). This is checked, not forced.
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0) atomicOr(err, OMNIA_ERR_TIMEOUT);
    return;
  }
  unsigned char* q_s = smem_raw;
  unsigned char* k_s = q_s + Q_BYTES;            // K_STAGES tiles of keys
  unsigned char* v_s = k_s + K_STAGES * K_BYTES;  // V_STAGES stages of values
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + V_STAGES * V_BYTES);
  // bars: q_full | k_full[K_STAGES] | v_full[V_STAGES] | v_done[V_STAGES] | s_full[S_BUFS] | p_full[S_BUFS] | p_done[S_BUFS] | g_full
  constexpr int BARS = 2 + K_STAGES + 2 * V_STAGES + 3 * S_BUFS;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile uint32_t* group_mask = reinterpret_cast<volatile uint32_t*>(tmem_holder + 2);  // [V_STAGES]
  // What the two threads of a row tell one another: a tile's maximum over their keys (two tiles' worth,
  // taking turns), and at the end their sums.
  float* row_state = reinterpret_cast<float*>(tmem_holder + 4 + V_STAGES);  // [2][128]: the offset each team last chose
  float* row_sum = row_state + 2 * BM;                                       // [2][128] sums, then [2][128] their offsets

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* item = work + WORK_INTS * blockIdx.x;
  const int seq = item[0], tok0 = item[1], kvh = item[2];
  if (item[4] >= 0 || (item[5] & 255) > 1) {  // a part of a block: not this kernel's
    if (threadIdx.x == 0) atomicOr(err, OMNIA_ERR_WORK);
    return;
  }
  const int q_begin = cu_seqlens[seq], q_len = cu_seqlens[seq + 1] - q_begin;
  const int pos0 = seq_lens[seq] - q_len + tok0;      // position of the block's first token
  const int tokens = min(TOKENS, q_len - tok0);
  const int rows = tokens * GROUP;
  const int last = pos0 + tokens - 1;                                   // last key any row sees
  const int first = window > 0 ? max(0, pos0 - window + 1) : 0;         // first key any row sees
  const int tile0 = first / BN;                                         // in units of BN keys
  const int n_tiles = last / BN - tile0 + 1;                            // V stages
  const int n_super = (n_tiles + HALVES - 1) / HALVES;                  // score tiles

  const uint32_t bar0 = smem_u32(bars);
  const uint32_t q_full = bar0, k_full0 = bar0 + 8, v_full0 = k_full0 + 8 * K_STAGES, v_done0 = v_full0 + 8 * V_STAGES,
                 s_full0 = v_done0 + 8 * V_STAGES, p_full0 = s_full0 + 8 * S_BUFS, p_done0 = p_full0 + 8 * S_BUFS,
                 g_full = p_done0 + 8 * S_BUFS;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < K_STAGES; ++s) mbar_init(k_full0 + 8 * s, 1);
    for (int s = 0; s < V_STAGES; ++s) mbar_init(v_full0 + 8 * s, 1), mbar_init(v_done0 + 8 * s, 1);
    for (int s = 0; s < S_BUFS; ++s) mbar_init(s_full0 + 8 * s, 1), mbar_init(p_full0 + 8 * s, 128), mbar_init(p_done0 + 8 * s, 1);
    mbar_init(g_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == WARP_QK) {
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

  if ((warp >= WARP_K && warp < WARP_K + FEEDERS) || (warp >= WARP_V && warp < WARP_V + FEEDERS)) {
    // ---- producers. Issuing a box (16 keys x 64 dims, a page group) keeps a warp busy for about
    // 70 ns whatever its size, so each ring has two warps that take turns with its stages. ----------
    const int which = warp >= WARP_V ? 1 : 0;          // 0 keys, 1 values
    const int turn = warp - (which ? WARP_V : WARP_K);  // this warp's stages: turn, turn + 2, ...
    if (warp == WARP_K && lane == 0) {
      mbar_expect_tx(q_full, DH * ROWS * 128);
      for (int h = 0; h < DH; ++h)
        tma_load_3d(smem_u32(q_s) + h * HALF_BYTES, &map_q, q_full, h * 64, kvh * GROUP, q_begin + tok0);
    }
    // Lane = group * DH + half: each of the stage's boxes is issued by its own lane.
    const int* table = block_table + (size_t)seq * max_pages;
    if (lane == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
    const int keys = which ? BN : SN;              // keys per stage of this ring
    const int count = which ? n_tiles : n_super;   // stages the ring's warps fill
    const int stages = which ? V_STAGES : K_STAGES;
    const int g = lane / DH, h = lane % DH;
    const bool active = lane < (keys / 16) * DH;
    // The page of this lane's group in stage t (-2: the group lies outside what the block reads).
    // Page numbers are fetched a turn before they are used, so the table's latency is hidden.
    auto lookup = [&](int t) {
      const int pos = tile0 * BN + t * keys + g * 16;
      return (active && t < count && pos <= last && pos + 15 >= first) ? table[pos / page_size] : -2;
    };
    bool ok = true;
    int issued = turn - FEEDERS;  // the last stage this warp has asked for
    auto load_stage = [&](int j, int page) {
      // A K stage is free when the scores computed from it are there (s_full of the same index: there
      // are as many score buffers as K stages), a V stage when its product is done (v_done).
      const int s = j % stages;
      const uint32_t full = (which ? v_full0 : k_full0) + 8 * s, empty = (which ? v_done0 : s_full0) + 8 * s;
      if (lane == 0 && j >= stages) ok = mbar_wait(empty, ((j / stages) & 1) ^ 1, abort_flag);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return;
      if (lane == 0) STAMP(0, j, which * 2);
      const int pos = tile0 * BN + j * keys + g * 16;
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
        const uint32_t dst = smem_u32(which ? v_s + s * V_BYTES : k_s + s * K_BYTES) + h * (which ? TILE_HALF : K_TILE_HALF) +
                             g * GROUP_BYTES;
        tma_load_2d(dst, &map_kv, full, h * 64, y);
      }
      if (lane == 0) STAMP(0, j, which * 2 + 1);
      issued = j;
    };
    int page_cur = lookup(turn);
    for (int j = turn; j < count && ok; j += FEEDERS) {
      const int page_next = lookup(j + FEEDERS);
      load_stage(j, page_cur);
      page_cur = page_next;
    }
    if (lane == 0 && *abort_flag) {
      // Giving up: what this warp has asked for must land before the block's shared memory goes away.
      const uint32_t full0 = which ? v_full0 : k_full0;
      for (int j = max(turn, issued - stages + FEEDERS); j <= issued; j += FEEDERS)
        for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(full0 + 8 * (j % stages), (j / stages) & 1); ++i) {
        }
      for (uint32_t i = 0; warp == WARP_K && i < WAIT_LIMIT && !mbar_try(q_full, 0); ++i) {
      }
    }
  } else if (warp == WARP_QK) {
    // ---- issuer of the score products: S[j & 1] = Q K_j^T, 128 keys a tile ----------------------------
    // A product with the 128-row operand in shared memory occupies the tensor core for 65 to 80 ns
    // however few columns it has, so a tile of 128 keys costs the eight products that a tile of 64
    // did. The two kinds of product are issued by two threads (this warp and the next), so the scores'
    // chain and the values' chain run side by side. What one thread's products must wait for of the
    // other's goes through barriers: a score buffer is written again only when the products that read
    // P from it are done (v_done of its last V stage, two tiles back).
    if (lane == 0) {
      constexpr uint32_t instr_s = idesc(BM, SN, false);
      // Descriptors differ only in their address field (the low 14 bits, in units of 16 bytes).
      const uint64_t q_desc = desc_k_major(smem_u32(q_s));
      uint64_t k_desc[K_STAGES];
      for (int s = 0; s < K_STAGES; ++s) k_desc[s] = desc_k_major(smem_u32(k_s + s * K_BYTES));
      bool ok = mbar_wait(q_full, 0, abort_flag);
      for (int j = 0; j < n_super && ok; ++j) {
        const int s = j % K_STAGES;
        ok = mbar_wait(k_full0 + 8 * s, (j / K_STAGES) & 1, abort_flag);
        // The buffer's last P has been read (p_done, S_BUFS tiles back; a V stage's own barrier
        // would not do: its ring comes round before the score buffers do).
        if (ok && j >= S_BUFS) ok = mbar_wait(p_done0 + 8 * s, ((j / S_BUFS) & 1) ^ 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        STAMP(1, j, 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma(tmem_base + S_COL + s * SN, q_desc + (((kk / 4) * HALF_BYTES + (kk % 4) * 32) >> 4),
               k_desc[s] + (((kk / 4) * K_TILE_HALF + (kk % 4) * 32) >> 4), instr_s, kk != 0);
        umma_commit(s_full0 + 8 * s);  // the scores are there, and with them the K stage is free again
        STAMP(1, j, 3);
      }
    }
  } else if (warp == WARP_PV) {
    // ---- issuer of the value products: O += P V, a V stage (64 keys) at a time ------------------------
    if (lane == 0) {
      constexpr uint32_t instr_o = idesc(BM, D, true);
      uint64_t v_desc[V_STAGES];
      for (int s = 0; s < V_STAGES; ++s) v_desc[s] = desc_mn_major(smem_u32(v_s + s * V_BYTES), TILE_HALF);
      uint32_t accumulate = 0;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % V_STAGES, tile = j / HALVES, b = tile % S_BUFS;
        ok = mbar_wait(v_full0 + 8 * s, (j / V_STAGES) & 1, abort_flag) &&
             mbar_wait(p_full0 + 8 * b, (tile / S_BUFS) & 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        STAMP(1, j, 1);
        const uint32_t mask = group_mask[s];
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          if (!(mask & (1u << kk))) continue;  // keys never loaded: their P is zero, their V is stale
          // P: 16 keys are eight columns of packed bfloat16 pairs, in the place of those keys' first eight scores
          umma_ts(tmem_base + O_COL, tmem_base + S_COL + b * SN + (j % HALVES) * BN + kk * 16,
                  v_desc[s] + ((kk * GROUP_BYTES) >> 4), instr_o, accumulate);
          accumulate = 1;
        }
        umma_commit(v_done0 + 8 * s);  // the product is done: the V stage is free, and O may be read or rescaled
        if (j % HALVES == HALVES - 1 || j == n_tiles - 1) umma_commit(p_done0 + 8 * b);  // and the tile's P has been read
        STAMP(1, j, 2);
      }
    }
  } else if (warp >= WARP_SOFTMAX && warp < WARP_SOFTMAX + 8) {
    // ---- softmax and epilogue: two teams of four warps, a thread per row in each. The teams take
    // turns with the score tiles (team 0 the even ones, team 1 the odd ones), so one team's
    // exponentials (the special-function unit sets the softmax's pace: an exponential and half a
    // conversion per score) run while the other reads its scores, finds its maximum and stores its
    // P. What a tile needs from the tile before is the exponent's offset only: it goes through shared
    // memory behind a pair of named barriers, right after the maximum is known. Each team keeps a sum
    // of its own, against the offset it last used; the two are brought together at the end. The warps
    // meet at the named barriers once a tile whatever `ok` says. -------------------------------------
    static_assert(THREADS == 32 * (WARP_V + FEEDERS), "every warp has one role");
    const int team = (warp - WARP_SOFTMAX) / 4;
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
    float m = -INFINITY, l = 0.f;  // the offset this team last used (in units of scores), its sum against it
    bool ok = true, gate_issued = false;
    const int tail = last / BN - tile0;  // the V stage that holds the block's last key
    for (int j = team; j < n_super; j += 2) {
      const int key0 = tile0 * BN + j * SN, b = j % S_BUFS;
      // (`ok` is kept the same for a warp's threads: what follows has warp-wide instructions.)
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(s_full0 + 8 * b, (j / S_BUFS) & 1, abort_flag));
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (ok && j == n_super - 1 && row == 0 && gate_tma) {
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
      const uint32_t s_addr = tmem_base + lane_field + S_COL + b * SN;
      // Which keys of the tile this row sees; a tile that the whole warp sees whole needs no masks.
      const int lo = max(row_lo - key0, 0), hi = min(row_hi - key0, SN - 1);  // visible columns [lo, hi]
      const bool unmasked = __all_sync(0xffffffffu, lo == 0 && hi == SN - 1);
      // First pass: the row's maximum over the tile, 32 scores at a time. (Read whatever `ok` says: a
      // block that is giving up reads columns that are its own all the same.)
      float tile_max = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < SN; c += 32) {
        uint32_t v[32];
        tmem_load32(s_addr + c, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (unmasked) {
          float part4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains instead of one
#pragma unroll
          for (int i = 0; i < 32; ++i) part4[i & 3] = fmaxf(part4[i & 3], __uint_as_float(v[i]));
          tile_max = fmaxf(tile_max, fmaxf(fmaxf(part4[0], part4[1]), fmaxf(part4[2], part4[3])));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c + i >= lo && c + i <= hi) tile_max = fmaxf(tile_max, __uint_as_float(v[i]));
        }
      }
      // The offset the tile before used (the other team's), then this tile's: the offset of the
      // exponent follows the row's maximum lazily. A softmax does not care which offset it is
      // computed with, so it moves only when the maximum has outgrown it by more than
      // 2^RESCALE_STEP (P then stays below that), and only then is the accumulator rescaled.
      if (j > 0) asm volatile("bar.sync %0, 256;" ::"r"(2 + (team ^ 1)) : "memory");
      const float before_m = j > 0 ? row_state[(team ^ 1) * BM + row] : -INFINITY;
      float now_m = before_m;
      float alpha = 1.f;
      if (tile_max > before_m) {
        if (before_m == -INFINITY) {
          now_m = tile_max;  // the row's first keys: nothing has been accumulated yet
        } else if ((tile_max - before_m) * sl2 > RESCALE_STEP) {
          alpha = fast_exp2((before_m - tile_max) * sl2);
          now_m = tile_max;
        }
      }
      row_state[team * BM + row] = now_m;
      if (j + 1 < n_super) asm volatile("bar.arrive %0, 256;" ::"r"(2 + team) : "memory");
      if (row == 0) STAMP(2, j, 1);
      if (!ok) continue;
      // This team's sum, brought to the new offset.
      if (now_m != m) {
        if (m != -INFINITY) l *= fast_exp2((m - now_m) * sl2);
        m = now_m;
      }
      if (__any_sync(0xffffffffu, alpha != 1.f)) {
        // The products so far must be done before the accumulator is rescaled. (The tile after this
        // one may rescale it too, but only behind this tile's products, which wait for this thread.)
        if (j > 0) {
          const int before = j * HALVES - 1;
          ok = __all_sync(0xffffffffu, mbar_wait(v_done0 + 8 * (before % V_STAGES), (before / V_STAGES) & 1, abort_flag));
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
#pragma unroll 1
        for (int c = 0; ok && c < D; c += 32) {
          uint32_t o[32];
          tmem_load32(tmem_base + lane_field + O_COL + c, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_store32(tmem_base + lane_field + O_COL + c, o);
        }
        if (!ok) continue;
      }
      if (row == 0) STAMP(2, j, 2);
      // Second pass: P = exp2(s * scale * log2e - offset), rounded to bfloat16, 32 scores at a time.
      // The pairs of 16 keys take the place of the first eight of those keys' scores, so nothing is
      // written over a score that has yet to be read. (This buffer's next scores are S_BUFS tiles
      // away, and their product is issued after this tile's P V.)
      const float offset = m == -INFINITY ? 0.f : m * sl2;
      float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
      for (int c = 0; c < SN; c += 32) {
        uint32_t v[32], packed[16];
        tmem_load32(s_addr + c, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (unmasked) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), sl2, -offset));
            const float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), sl2, -offset));
            sums[(i >> 1) & 3] += p0 + p1;
            packed[i / 2] = pack_bf16(p0, p1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int col = c + i + e;
              p[e] = (col >= lo && col <= hi) ? fast_exp2(fmaf(__uint_as_float(v[i + e]), sl2, -offset)) : 0.f;
            }
            sums[(i >> 1) & 3] += p[0] + p[1];
            packed[i / 2] = pack_bf16(p[0], p[1]);
          }
        }
        tmem_store8(s_addr + c, packed);
        tmem_store8(s_addr + c + 16, packed + 8);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      l += (sums[0] + sums[1]) + (sums[2] + sums[3]);
      if (tail >= j * HALVES && tail < min((j + 1) * HALVES, n_tiles) && ((last + 1) & 15)) {
        // The last group of 16 keys reaches past the block's last key. Those rows of V get a
        // zero weight, but what they hold need not be a number: past the request's last token
        // the page still holds whatever its previous owner left (0 x NaN is NaN). Clear them in
        // the stage once it has landed; the fence orders the stores before the P V product.
        const int s = tail % V_STAGES;
        ok = __all_sync(0xffffffffu, mbar_wait(v_full0 + 8 * s, (tail / V_STAGES) & 1, abort_flag));
        if (!ok) continue;
        const int r0 = last - (tile0 + tail) * BN + 1, r1 = (r0 + 15) & ~15;  // rows [r0, r1) of the stage
        unsigned char* v_tile = v_s + s * V_BYTES;
        for (int i = row; i < (r1 - r0) * DH * 8; i += 128) {
          const int piece = i & 7, h = (i >> 3) % DH, r = r0 + (i >> 3) / DH;
          *reinterpret_cast<uint4*>(v_tile + h * TILE_HALF + r * 128 + piece * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // V is read by the tensor core (async proxy)
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(p_full0 + 8 * b);
      if (row == 0) STAMP(2, j, 3);
      if (lane == 0) STAMP(3, j, quarter);
    }
    // Epilogue: O / l, gate, store; the row's thread of team 0 has the first half of its dims, that of
    // team 1 the second. A thread owns a row, so a warp's loads and stores go to 32 different rows,
    // each a trip to L2 of its own: read that way (two bytes at a time, then sixteen) the gate cost a
    // block 30 and 13 us. It comes by TMA into Q's place instead (see the loop) and is read from
    // shared memory, 16 bytes at a time, like everything stored.
    OMNIA_TRACE_IF(row == 0 && team == 0, 6);
    constexpr int MY_DIMS = D / 2;
    const int c0 = team * MY_DIMS;
    const size_t token = (size_t)(q_begin + tok0 + row / GROUP);
    const int head = kvh * GROUP + row % GROUP;
    const bf16* gp = gate ? gate + token * gate_stride + (size_t)head * D : nullptr;
    const bool gate_wide = gp != nullptr && (reinterpret_cast<uintptr_t>(gp) & 15) == 0;
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(v_done0 + 8 * ((n_tiles - 1) % V_STAGES), ((n_tiles - 1) / V_STAGES) & 1, abort_flag));
    if (ok && gate_tma) ok = __all_sync(0xffffffffu, mbar_wait(g_full, 0, abort_flag));
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // The row's sum: the teams' sums brought to the last offset (the last tile's), team 0's first.
    row_sum[team * BM + row] = l;
    row_sum[(2 + team) * BM + row] = m;
    softmax_sync();
    m = row_state[((n_super - 1) & 1) * BM + row];
    l = 0.f;
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      const float its_m = row_sum[(2 + x) * BM + row];
      if (its_m != -INFINITY) l += row_sum[x * BM + row] * fast_exp2((its_m - m) * sl2);
    }
    OMNIA_TRACE_IF(row == 0 && team == 0, 7);
    if (ok) {
      // The thread's half of the row's accumulator in one go (a load from tensor memory takes some
      // 0.35 us to arrive: eight dims a turn with the next turn's columns on their way took a block
      // 3.2 us here), then eight dims a turn: normalise, gate, 16 bytes stored.
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = out + (token * nq + head) * D;
      const uint32_t o_addr = tmem_base + lane_field + O_COL + c0;
      static_assert(MY_DIMS == 32 || MY_DIMS == 64, "a thread's dims are one or two loads of 32 columns");
      uint32_t acc[MY_DIMS];
#pragma unroll
      for (int c = 0; c < MY_DIMS; c += 32) tmem_load32(o_addr + c, acc + c);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (live) {
#pragma unroll
        for (int i = 0; i < MY_DIMS; i += 8) {
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
    } else if (gate_issued) {
      // Giving up: the gate's copy must land before the block's shared memory goes away.
      for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try(g_full, 0); ++i) {
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  OMNIA_TRACE_BLOCK(4);
  if (warp == WARP_QK) {
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

extern "C" int omnia_attention_tcgen05_info(int* head_dim, int* group, int* tokens_per_block) {
  *head_dim = HEAD_DIM;
  *group = GROUP;
  *tokens_per_block = TOKENS;
  return 0;
}

// q: [tokens, nq, D]; pages: [num_pages, 2, nkv, page_size, D]; page_size a multiple of 16.
// work: `blocks` items of 8 ints (see the kernel).
extern "C" int omnia_attention_prefill_tcgen05_wide(const void* q, int tokens, const void* pages, const int* block_table,
                                               const int* cu_seqlens, const int* seq_lens, const int* work,
                                               int blocks, const void* gate, int gate_stride, void* out,
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
  constexpr size_t smem = Q_BYTES + K_STAGES * K_BYTES + V_STAGES * V_BYTES + 256 + 6 * BM * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  launch_pdl(attention_prefill_tcgen05_kernel, blocks, THREADS, smem, stream,
             map_q, map_kv, map_gate, gate_tma, block_table, cu_seqlens, seq_lens, work, (const bf16*)gate, gate_stride, (bf16*)out,
             max_pages, num_pages, nq, nkv, page_size, window, scale, err);
  return OMNIA_LAUNCH_RESULT();
}
