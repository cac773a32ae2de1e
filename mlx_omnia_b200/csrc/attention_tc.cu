// Paged causal attention in bfloat16 on the tensor cores (mma.sync m16n8k16, float32
// accumulation and softmax), compiled for one head size and one group size:
//   -DHEAD_DIM=d   (a multiple of 8, at most 256; rows are zero-padded to a multiple of 16)
//   -DGROUP=g      (query heads per key/value head, at most 16)
//
// Rows of a tile are (token, query head of the group) pairs of ONE key/value head, so a
// key/value tile fetched from the cache serves the whole group. Two kernels share the
// tile arithmetic:
//   prefill:  a block of 4 warps owns 64 rows (64 / g tokens of one request) and walks
//             the visible keys in tiles of 64, double-buffered with cp.async; it writes
//             the final output (optionally times sigmoid(gate)).
//   decode:   one warp per block owns the g rows of one single-token request and one
//             chunk of keys (chunks are aligned to absolute key positions; the caller picks
//             their size from the number of requests and the longest one); it writes an
//             unnormalised partial (max, sum, accumulator) to scratch memory and takes a
//             ticket; the block that draws the last ticket of a (request, head group)
//             merges that group's chunks in ascending order (nobody waits for anybody).
// Keys and values are addressed row by row through the block table, so any page size
// works. Rows outside the visible range are zero-filled in shared memory (never read
// from the cache), which keeps stale or poisoned pages out of the arithmetic.
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
#ifndef GROUP
#define GROUP 2
#endif

namespace {

constexpr int D = HEAD_DIM;
constexpr int DP = (D + 15) / 16 * 16;   // padded head size
constexpr int ROW = DP + 8;              // shared-memory row stride (elements): odd in 16-byte units
constexpr int CH = D / 8;                // 16-byte chunks of a stored row
constexpr int CHP = DP / 8;              // 16-byte chunks of a padded row
constexpr int KSTEPS = DP / 16;
constexpr int NT_O = DP / 8;             // output n-tiles
constexpr int BM = 64;                   // rows per prefill block
constexpr int BN = 64;                   // keys per prefill tile
constexpr int TOKENS_PER_BLOCK = BM / GROUP;
#ifndef DECODE_TILE_KEYS
#define DECODE_TILE_KEYS 32
#endif
#ifndef DECODE_PIPELINE
#define DECODE_PIPELINE 2
#endif
constexpr int DECODE_BN = DECODE_TILE_KEYS;   // keys per decode tile
static_assert(DECODE_TILE_KEYS == 32, "a decode tile is loaded by one warp, lane l looking up key l: 32 keys");
constexpr int DECODE_STAGES = DECODE_PIPELINE;
constexpr int DECODE_TABLE = 64;         // block-table entries a decode block stages in shared memory
constexpr float LOG2E = 1.4426950408889634f;

static_assert(D % 8 == 0 && D <= 256, "head size must be a multiple of 8, at most 256");
static_assert(GROUP >= 1 && GROUP <= 16, "group size must be 1..16");

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3,
                                            const bf16* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2,
                                                  unsigned& r3, const bf16* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

struct CacheRef {
  const bf16* pages;   // [num_pages, 2, nkv, page_size, D]
  const int* table;    // block-table entries, entry 0 being logical page `first_page`
  int first_page, num_pages, nkv, kvh, page_size;
};

// The address of key (which = 0) or value (which = 1) row `pos`; null when its page is bad.
__device__ __forceinline__ const bf16* cache_row(const CacheRef& c, int pos, int which, int* err) {
  const int logical = pos / c.page_size;
  const int page = c.table[logical - c.first_page];
  if (page < 0 || page >= c.num_pages) {
    atomicOr(err, OMNIA_ERR_PAGE);
    return nullptr;
  }
  return c.pages + ((((size_t)page * 2 + which) * c.nkv + c.kvh) * c.page_size + (pos - logical * c.page_size)) * D;
}

// One tile of the online softmax for the 16 rows of a warp.
//   qf:      the warp's query fragments (KSTEPS x 4 registers)
//   ks, vs:  shared-memory tiles [NKEYS][ROW]
//   key0:    absolute position of the tile's first key
//   row_lo/row_hi[2]: visible key range of the warp's rows g and g + 8 (inclusive; lo > hi: none)
template <int NKEYS>
__device__ __forceinline__ void attend_tile(const unsigned (*qf)[4], const bf16* ks, const bf16* vs,
                                            int key0, const int* row_lo, const int* row_hi,
                                            float sl2, float* m, float* l, float (*o)[4]) {
  const int lane = threadIdx.x & 31;
  const int t = lane & 3;
  constexpr int NT = NKEYS / 8;
  float s[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
  for (int kstep = 0; kstep < KSTEPS; ++kstep) {
#pragma unroll
    for (int j2 = 0; j2 < NT / 2; ++j2) {
      unsigned b0, b1, b2, b3;
      const int mat = lane >> 3;
      ldmatrix_x4(b0, b1, b2, b3,
                  ks + (j2 * 16 + (mat >> 1) * 8 + (lane & 7)) * ROW + kstep * 16 + (mat & 1) * 8);
      mma_bf16(s[2 * j2], qf[kstep], b0, b1);
      mma_bf16(s[2 * j2 + 1], qf[kstep], b2, b3);
    }
  }
  // Mask, then the running maximum of rows g (elements 0,1) and g + 8 (elements 2,3).
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key0 + 8 * j + 2 * t + (e & 1);
      const int r = e >> 1;
      if (key < row_lo[r] || key > row_hi[r]) s[j][e] = -INFINITY;
      mx[r] = fmaxf(mx[r], s[j][e]);
    }
  }
  float alpha[2], base[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float m_new = fmaxf(m[r], mx[r]);
    base[r] = m_new == -INFINITY ? 0.f : m_new * sl2;
    alpha[r] = m[r] == -INFINITY ? 0.f : exp2f(m[r] * sl2 - base[r]);
    m[r] = m_new;
    l[r] *= alpha[r];
  }
#pragma unroll
  for (int j = 0; j < NT_O; ++j) {
    o[j][0] *= alpha[0];
    o[j][1] *= alpha[0];
    o[j][2] *= alpha[1];
    o[j][3] *= alpha[1];
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p = exp2f(s[j][e] * sl2 - base[e >> 1]);  // exp2(-inf) = 0 for masked keys
      s[j][e] = p;
      l[e >> 1] += p;
    }
  }
#pragma unroll
  for (int kk = 0; kk < NKEYS / 16; ++kk) {
    unsigned a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int j2 = 0; j2 < NT_O / 2; ++j2) {
      unsigned b0, b1, b2, b3;
      const int mat = lane >> 3;
      ldmatrix_x4_trans(b0, b1, b2, b3,
                        vs + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * ROW + j2 * 16 + (mat >> 1) * 8);
      mma_bf16(o[2 * j2], a, b0, b1);
      mma_bf16(o[2 * j2 + 1], a, b2, b3);
    }
  }
}

// Load the warp's 16 query rows as A fragments. qs: [16 or more rows][ROW].
__device__ __forceinline__ void load_q_fragments(const bf16* qs, unsigned (*qf)[4]) {
  const int lane = threadIdx.x & 31, mat = lane >> 3;
#pragma unroll
  for (int kstep = 0; kstep < KSTEPS; ++kstep)
    ldmatrix_x4(qf[kstep][0], qf[kstep][1], qf[kstep][2], qf[kstep][3],
                qs + ((mat & 1) * 8 + (lane & 7)) * ROW + kstep * 16 + (mat >> 1) * 8);
}

// Zero the padding chunks (dims D..DP-1) of `rows` shared-memory rows.
__device__ __forceinline__ void zero_padding(bf16* tile, int rows, int tid, int threads) {
  if (CHP != CH) {
    constexpr int PAD = CHP != CH ? CHP - CH : 1;
    for (int i = tid; i < rows * PAD; i += threads) {
      const int r = i / PAD, c = CH + i % PAD;
      *reinterpret_cast<uint4*>(tile + r * ROW + c * 8) = make_uint4(0, 0, 0, 0);
    }
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------
// Prefill: grid (blocks of the work list, nkv); 128 threads.
__global__ void __launch_bounds__(128)
attention_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pages,
                         const int* __restrict__ block_table, const int* __restrict__ cu_seqlens,
                         const int* __restrict__ seq_lens, const int* __restrict__ work,
                         const bf16* __restrict__ gate, int gate_stride, bf16* __restrict__ out,
                         int max_pages, int num_pages, int nq, int nkv, int page_size, int window,
                         float scale, int* err) {
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);   // [BM][ROW]
  bf16* kv = qs + BM * ROW;                       // 2 stages x (K [BN][ROW], V [BN][ROW])
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq = work[2 * blockIdx.x], tok0 = work[2 * blockIdx.x + 1];
  const int kvh = blockIdx.y;
  const int q_begin = cu_seqlens[seq], q_len = cu_seqlens[seq + 1] - q_begin;
  const int pos0 = seq_lens[seq] - q_len + tok0;  // position of the block's first token
  const int tokens = min(TOKENS_PER_BLOCK, q_len - tok0);
  const int rows = tokens * GROUP;
  CacheRef cache{pages, block_table + (size_t)seq * max_pages, 0, num_pages, nkv, kvh, page_size};

  // Query rows: row r = (token r / GROUP, head kvh * GROUP + r % GROUP).
  for (int i = tid; i < BM * CHP; i += 128) {
    const int r = i / CHP, c = i % CHP;
    const bool valid = r < rows && c < CH;
    const bf16* src = q + ((size_t)(q_begin + tok0 + r / GROUP) * nq + kvh * GROUP + r % GROUP) * D + c * 8;
    cp_async16(qs + r * ROW + c * 8, valid ? src : q, valid);
  }
  cp_async_commit();
  for (int stage = 0; stage < 2; ++stage) {
    zero_padding(kv + stage * 2 * BN * ROW, 2 * BN, tid, 128);
  }

  const int last = pos0 + tokens - 1;                                    // last key any row sees
  const int first = window > 0 ? max(0, pos0 - window + 1) : 0;          // first key any row sees
  const int tile0 = first / BN, tiles = last / BN - tile0 + 1;

  auto load_tile = [&](int tile, int stage) {
    bf16* kt = kv + stage * 2 * BN * ROW;
    bf16* vt = kt + BN * ROW;
    const int key = tid >> 1, sub = tid & 1;
    const int pos = (tile0 + tile) * BN + key;
    const bool visible = pos >= first && pos <= last;
    const bf16* kp = visible ? cache_row(cache, pos, 0, err) : nullptr;
    const bf16* vp = kp ? kp + (size_t)nkv * page_size * D : nullptr;
#pragma unroll
    for (int c = sub; c < CH; c += 2) {
      cp_async16(kt + key * ROW + c * 8, kp ? kp + c * 8 : pages, kp != nullptr);
      cp_async16(vt + key * ROW + c * 8, vp ? vp + c * 8 : pages, kp != nullptr);
    }
  };

  load_tile(0, 0);
  cp_async_commit();

  unsigned qf[KSTEPS][4];
  float o[NT_O][4];
#pragma unroll
  for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  // Visible key range of this lane's two rows.
  int row_lo[2], row_hi[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + (lane >> 2) + 8 * r;
    const int pos = pos0 + row / GROUP;
    row_hi[r] = row < rows ? pos : -1;
    row_lo[r] = row < rows ? (window > 0 ? max(0, pos - window + 1) : 0) : 0;
  }
  const float sl2 = scale * LOG2E;

  for (int tile = 0; tile < tiles; ++tile) {
    if (tile + 1 < tiles) load_tile(tile + 1, (tile + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (tile == 0) load_q_fragments(qs + warp * 16 * ROW, qf);
    const bf16* kt = kv + (tile & 1) * 2 * BN * ROW;
    // A warp whose rows see nothing of this tile skips it (rows are ordered by position).
    const int key0 = (tile0 + tile) * BN;
    const int warp_last = pos0 + min(rows - 1, warp * 16 + 15) / GROUP;
    if (warp * 16 < rows && key0 <= warp_last)
      attend_tile<BN>(qf, kt, kt + BN * ROW, key0, row_lo, row_hi, sl2, m, l, o);
    __syncthreads();
  }
  cp_async_wait<0>();
  pdl_launch_dependents();  // the cache is read: the next kernel may begin its preamble

  // Normalise, gate, store.
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  const int t = lane & 3;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + (lane >> 2) + 8 * r;
    if (row >= rows) continue;
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
    const size_t token = (size_t)(q_begin + tok0 + row / GROUP);
    const int head = kvh * GROUP + row % GROUP;
    bf16* dst = out + (token * nq + head) * D;
    const bf16* gp = gate ? gate + token * gate_stride + (size_t)head * D : nullptr;
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
      const int dim = 8 * j + 2 * t;
      if (dim >= D) continue;
      float v0 = o[j][2 * r] * inv, v1 = o[j][2 * r + 1] * inv;
      if (gp) {
        v0 *= 1.f / (1.f + expf(-__bfloat162float(gp[dim])));
        v1 *= 1.f / (1.f + expf(-__bfloat162float(gp[dim + 1])));
      }
      *reinterpret_cast<__nv_bfloat162*>(dst + dim) = __floats2bfloat162_rn(v0, v1);
    }
  }
}

// Merge chunks c0..c1 of H heads of one token (heads head0 .., whose partials lie max_chunks apart),
// ascending, then gate and round; run by one warp. The merge is the tail of the whole kernel and
// nothing but memory round trips (the partials were written to L2 a moment ago by other blocks), so
// everything a round needs is asked for before anything is used: the gates at once, then per
// round of eight chunks the chunks' (max, sum) pairs, one chunk per lane, and the H x 8 partial
// rows, every lane its own dims. Eight chunks or fewer are one round trip for all H heads.
// The merge of a head's (H heads') chunks by one warp. The chunks' unnormalised accumulators lie one
// after the other in part_o, so a batch of them is brought into shared memory (`stage`, room for
// `stage_floats` floats: the block's ring, idle by now) with one round of 16-byte asynchronous
// copies, all in flight together: one trip to L2 for up to 32 chunks, where reading them eight at
// a time into registers took one trip per eight. Lane u holds chunk u's maximum and sum.
template <int H>
__device__ __forceinline__ void combine_heads(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              size_t base, int max_chunks, int c0, int c1, const bf16* gate_row,
                                              bf16* out_row, float* stage, int stage_floats) {
  const int lane = threadIdx.x & 31;
  constexpr int PER_LANE = (D + 31) / 32;
  float gate_v[H][PER_LANE];
#pragma unroll
  for (int h = 0; h < H; ++h)
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
      const int dim = lane + 32 * k;
      gate_v[h][k] = gate_row && dim < D ? __bfloat162float(gate_row[(size_t)h * D + dim]) : 0.f;
    }
  float acc[H][PER_LANE], mx[H], total[H];
#pragma unroll
  for (int h = 0; h < H; ++h) {
    mx[h] = -INFINITY, total[h] = 0.f;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) acc[h][k] = 0.f;
  }
  const int batch = min(32, stage_floats / (H * D));  // chunks a round (at least one: a stage holds far more than H rows)
  for (int r0 = c0; r0 <= c1; r0 += batch) {
    const int count = min(batch, c1 - r0 + 1);
    float mc[H], lc[H];
#pragma unroll
    for (int h = 0; h < H; ++h) {
      const size_t slot = base + (size_t)h * max_chunks + r0;
      const float* src = part_o + slot * D;  // `count` chunks of D floats, one after the other
      for (int i = lane; i < count * (D / 4); i += 32) cp_async16(stage + (size_t)h * batch * D + 4 * i, src + 4 * i, true);
      mc[h] = lane < count ? __ldcg(part_ml + (slot + lane) * 2) : -INFINITY;
      lc[h] = lane < count ? __ldcg(part_ml + (slot + lane) * 2 + 1) : 0.f;
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();
#pragma unroll
    for (int h = 0; h < H; ++h) {
      const float mx_new = fmaxf(mx[h], warp_max(mc[h]));
      const float rescale = mx[h] == -INFINITY ? 0.f : exp2f(mx[h] - mx_new);
      const float w = lane < count && mc[h] != -INFINITY ? exp2f(mc[h] - mx_new) : 0.f;
      total[h] = total[h] * rescale + warp_sum(lc[h] * w);
      mx[h] = mx_new;
#pragma unroll
      for (int k = 0; k < PER_LANE; ++k) acc[h][k] *= rescale;
      const float* rows = stage + (size_t)h * batch * D;
      for (int u = 0; u < count; ++u) {
        const float wj = __shfl_sync(0xffffffffu, w, u);
#pragma unroll
        for (int k = 0; k < PER_LANE; ++k) {
          const int dim = lane + 32 * k;
          if (dim < D) acc[h][k] += rows[u * D + dim] * wj;
        }
      }
    }
    __syncwarp();  // the stage is read before the next round overwrites it
  }
#pragma unroll
  for (int h = 0; h < H; ++h) {
    const float inv = total[h] > 0.f ? 1.f / total[h] : 0.f;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
      const int dim = lane + 32 * k;
      if (dim >= D) continue;
      float v = acc[h][k] * inv;
      if (gate_row) v *= 1.f / (1.f + expf(-gate_v[h][k]));
      out_row[(size_t)h * D + dim] = __float2bfloat16_rn(v);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Decode: grid (chunks, nkv, requests); WARPS x 32 threads. Request s is the single-token
// request seq_ids[s] (or s when seq_ids is null). With one warp the block walks its chunk's tiles
// through a two-stage ring; with four (small batches, where there are too few chunks to fill the
// GPU otherwise) the warps take the tiles in turn, one stage each, and their states are merged
// through shared memory before the block's partial is written. Partials:
//   part_o  [requests, nq, max_chunks, D] float32 (unnormalised), part_ml [requests, nq, max_chunks, 2]
//   tickets [requests, nkv] int32, zero before the first launch; the merging block zeroes its
//   ticket again, so the array is ready for the next launch.
// What the decode kernel needs to do the step before it as well (a decode step's QK-norm, rotation
// and cache write): the projected rows [.. q heads .. | .. k heads .. | .. v heads ..], each group
// at its own column; `proj` null means q is given and the cache already holds the new token.
struct FusedQK {
  const bf16* proj;
  int stride, q_col, k_col, v_col;
  float eps;                       // of the weightless RMS norm of every q and k head; < 0: none
  const float* inv_freq;           // D / 2 inverse frequencies (rotation of all D dims), or null
  const long long* slot_mapping;   // where each token's key and value go: page * page_size + offset
  bf16* pages;                     // the same pages, for writing
  long long num_slots;
};

template <int WARPS, int RING>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pages,
                        const int* __restrict__ block_table, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ seq_lens, const int* __restrict__ seq_ids,
                        float* __restrict__ part_o, float* __restrict__ part_ml,
                        int* __restrict__ tickets, const bf16* __restrict__ gate, int gate_stride,
                        bf16* __restrict__ out, int chunk_keys, int max_chunks, int max_pages,
                        int num_pages, int nq, int nkv, int page_size, int window, float scale,
                        const FusedQK fused, int* err) {
  // In the fused mode nothing up to the query fragments depends on the kernel before this one
  // (the lengths and tables were copied in before the step began, the keys and values of earlier
  // tokens were written in earlier steps), so the block's start and its first loads of the cache
  // run while that kernel finishes. Every block waits before it leaves, also one with nothing to do.
  const bool early = fused.proj != nullptr;
  OMNIA_TRACE_BLOCK(2);
  if (!early) pdl_wait();
  constexpr int STAGES = RING;  // stages of each warp's own ring
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  bf16* kv = reinterpret_cast<bf16*>(smem_raw) + warp * STAGES * 2 * DECODE_BN * ROW;  // STAGES x (K [32][ROW], V [32][ROW])
  const int seq = seq_ids ? seq_ids[blockIdx.z] : blockIdx.z;
  const int kvh = blockIdx.y, chunk = blockIdx.x;
  const int pos = seq_lens[seq] - 1;
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const int lo = max(first, chunk * chunk_keys), hi = min(pos, (chunk + 1) * chunk_keys - 1);
  if (pos < 0 || lo > hi) {
    if (early) pdl_wait();
    return;
  }
  const size_t token = (size_t)cu_seqlens[seq];
  // The chunk's block-table entries are read once, up front: a tile's loads then never wait
  // for a table lookup. (Chunks of more than DECODE_TABLE pages read the table directly.)
  __shared__ int table_s[DECODE_TABLE];
  const int page_lo = lo / page_size, page_hi = hi / page_size;
  const int* table_row = block_table + (size_t)seq * max_pages;
  const bool staged = page_hi - page_lo < DECODE_TABLE;
  if (staged)
    for (int i = threadIdx.x; i <= page_hi - page_lo; i += WARPS * 32) table_s[i] = table_row[page_lo + i];
  CacheRef cache{pages, staged ? table_s : table_row, staged ? page_lo : 0, num_pages, nkv, kvh, page_size};
  if (WARPS == 1) __syncwarp(); else __syncthreads();

  for (int stage = 0; stage < STAGES; ++stage)
    zero_padding(kv + stage * 2 * DECODE_BN * ROW, 2 * DECODE_BN, lane, 32);

  // This warp's tiles: every WARPS-th of the chunk's, starting with its own number.
  const int tile0 = lo / DECODE_BN + warp, all_tiles = hi / DECODE_BN - lo / DECODE_BN + 1;
  const int tiles = (all_tiles - warp + WARPS - 1) / WARPS;
  // A tile's loads: lane l looks up the row of key l once; then the warp copies the tile in
  // flat order (consecutive lanes take consecutive 16-byte chunks of a row, so every
  // request covers whole 128-byte lines), fetching each row's address by shuffle.
  auto load_tile = [&](int tile, int stage) {
    bf16* kt = kv + stage * 2 * DECODE_BN * ROW;
    bf16* vt = kt + DECODE_BN * ROW;
    const int p = (tile0 + tile * WARPS) * DECODE_BN + lane;
    const bool visible = p >= lo && p <= hi;
    const bf16* mine = visible ? cache_row(cache, p, 0, err) : nullptr;
    const size_t v_offset = (size_t)nkv * page_size * D;
#pragma unroll
    for (int it = 0; it < CH; ++it) {
      const int flat = it * 32 + lane;
      const int key = flat / CH, c = flat % CH;
      const bf16* kp = reinterpret_cast<const bf16*>(
          __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(mine), key));
      cp_async16(kt + key * ROW + c * 8, kp ? kp + c * 8 : pages, kp != nullptr);
      cp_async16(vt + key * ROW + c * 8, kp ? kp + v_offset + c * 8 : pages, kp != nullptr);
    }
  };
  // In flight before the loop: all stages but one of a lone warp's ring (the last is asked for at the
  // top of the loop), the one stage of a warp without a ring, every stage of a ring beside other
  // warps' (FILLED: a stage is then asked for again once its tile has been worked on).
  constexpr bool FILLED = WARPS > 1 && STAGES > 1;
  constexpr int AHEAD = FILLED ? STAGES : STAGES > 1 ? STAGES - 1 : 1;
#pragma unroll
  for (int s = 0; s < AHEAD; ++s) {
    if (s < tiles) load_tile(s, s);
    cp_async_commit();
  }

  // Query fragments straight from global memory: row g of the A operand is query head g of
  // the group (rows at or beyond GROUP are zero), columns 2t, 2t+1 (+8) of each 16-wide step.
  // In the fused mode they are read from the projected row, normalised and rotated here: a
  // thread holds 2 x 2 values of every 16 dims of heads g and g + 8, so a head's sum of squares
  // is a sum over the four threads of its row, and a dim's rotation partner (D / 2 further)
  // lies in the same thread, KSTEPS / 2 steps further.
  // The token's rotation angles, once per warp: cos of the D / 2 angles, then their sin.
  __shared__ float rope_cs[WARPS][D];
  if (fused.proj && fused.inv_freq) {
    for (int i = lane; i < D / 2; i += 32) sincosf((float)pos * fused.inv_freq[i], &rope_cs[warp][D / 2 + i], &rope_cs[warp][i]);
    __syncwarp();
  }
  OMNIA_TRACE_BLOCK(3);
  if (early) pdl_wait();
  OMNIA_TRACE_BLOCK(4);
  unsigned qf[KSTEPS][4];
  {
    const int g = lane >> 2, t = lane & 3;
    const bf16* q_src = fused.proj ? fused.proj + token * fused.stride + fused.q_col : q + token * nq * D;
#pragma unroll
    for (int kstep = 0; kstep < KSTEPS; ++kstep) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int dim = kstep * 16 + half * 8 + 2 * t;
        unsigned lo_row = 0u, hi_row = 0u;
        if (dim < D) {
          if (g < GROUP) lo_row = __ldcg(reinterpret_cast<const unsigned*>(q_src + (size_t)(kvh * GROUP + g) * D + dim));
          if (g + 8 < GROUP) hi_row = __ldcg(reinterpret_cast<const unsigned*>(q_src + (size_t)(kvh * GROUP + g + 8) * D + dim));
        }
        qf[kstep][2 * half] = lo_row;
        qf[kstep][2 * half + 1] = hi_row;
      }
    }
    if (fused.proj) {
      // v[row][kstep][half][e]: float32 copies of the fragment values.
      float ss[2] = {0.f, 0.f};
#pragma unroll
      for (int kstep = 0; kstep < KSTEPS; ++kstep)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qf[kstep][x]));
          ss[x & 1] += f.x * f.x + f.y * f.y;
        }
      float norm[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], 1);
        ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], 2);
        norm[r] = fused.eps >= 0.f ? rsqrtf(ss[r] / (float)D + fused.eps) : 1.f;
      }
#pragma unroll
      for (int kstep = 0; kstep < KSTEPS / 2; ++kstep)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          // Slot x of step kstep holds dims (kstep * 16 + (x >> 1) * 8 + 2 t, + 1) of row g + 8 * (x & 1).
          const int dim = kstep * 16 + (x >> 1) * 8 + 2 * t;
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qf[kstep][x]));
          const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qf[kstep + KSTEPS / 2][x]));
          const float n = norm[x & 1];
          float c0 = 1.f, s0 = 0.f, c1 = 1.f, s1 = 0.f;
          if (fused.inv_freq) {
            c0 = rope_cs[warp][dim], s0 = rope_cs[warp][D / 2 + dim];
            c1 = rope_cs[warp][dim + 1], s1 = rope_cs[warp][D / 2 + dim + 1];
          }
          const float ax = a.x * n, ay = a.y * n, bx = b.x * n, by = b.y * n;
          qf[kstep][x] = pack_bf16(ax * c0 - bx * s0, ay * c1 - by * s1);
          qf[kstep + KSTEPS / 2][x] = pack_bf16(ax * s0 + bx * c0, ay * s1 + by * c1);
        }
    }
  }
  // Fused mode: the new token's key and value (this request's, this head's), for the warp whose
  // tile holds position `pos`: lane l owns dims l * D / 32 .. of the head; a dim's rotation
  // partner lives 16 lanes away. They go to the cache pages and, once that tile has landed,
  // over its row of the tile (the cache had nothing there yet).
  constexpr int VW = D / 32 > 0 ? D / 32 : 1;
  float new_k[VW], new_v[VW];
  const bool brings_new = fused.proj != nullptr && pos >= lo && pos <= hi &&
                          ((pos / DECODE_BN - lo / DECODE_BN) % WARPS) == warp;
  if (brings_new) {
    const bf16* k_src = fused.proj + token * fused.stride + fused.k_col + (size_t)kvh * D + lane * VW;
    const bf16* v_src = fused.proj + token * fused.stride + fused.v_col + (size_t)kvh * D + lane * VW;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VW; ++i) {
      new_k[i] = __bfloat162float(k_src[i]);
      new_v[i] = __bfloat162float(v_src[i]);
      ss += new_k[i] * new_k[i];
    }
    const float n = fused.eps >= 0.f ? rsqrtf(warp_sum(ss) / (float)D + fused.eps) : 1.f;
#pragma unroll
    for (int i = 0; i < VW; ++i) {
      float mine = new_k[i] * n;
      if (fused.inv_freq) {
        const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
        const float c = rope_cs[warp][(lane & 15) * VW + i], sn = rope_cs[warp][D / 2 + (lane & 15) * VW + i];
        mine = lane < 16 ? mine * c - other * sn : other * sn + mine * c;
      }
      new_k[i] = __bfloat162float(__float2bfloat16_rn(mine));  // as the cache will hold it
    }
    const long long slot = fused.slot_mapping[token];
    if (slot >= 0 && slot < fused.num_slots) {
      const long long page = slot / page_size, off = slot % page_size;
      bf16* k_dst = fused.pages + (((page * 2 + 0) * nkv + kvh) * page_size + off) * D + lane * VW;
      bf16* v_dst = fused.pages + (((page * 2 + 1) * nkv + kvh) * page_size + off) * D + lane * VW;
#pragma unroll
      for (int i = 0; i < VW; ++i) {
        k_dst[i] = __float2bfloat16_rn(new_k[i]);
        v_dst[i] = __float2bfloat16_rn(new_v[i]);
      }
    } else if (slot >= fused.num_slots && lane == 0) {
      atomicOr(err, OMNIA_ERR_SLOT);
    }
  }
  float o[NT_O][4];
#pragma unroll
  for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  int row_lo[2], row_hi[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = (lane >> 2) + 8 * r;
    row_lo[r] = lo;
    row_hi[r] = row < GROUP ? hi : -1;
  }
  const float sl2 = scale * LOG2E;

  for (int tile = 0; tile < tiles; ++tile) {
    if (FILLED) {
      cp_async_wait<STAGES - 1>();
    } else if (STAGES > 1) {
      const int ahead = tile + STAGES - 1;
      if (ahead < tiles) load_tile(ahead, ahead % STAGES);
      cp_async_commit();
      cp_async_wait<STAGES - 1>();
    } else {
      cp_async_wait<0>();
    }
    __syncwarp();
    bf16* kt = kv + (tile % STAGES) * 2 * DECODE_BN * ROW;
    if (brings_new && (tile0 + tile * WARPS) == pos / DECODE_BN) {
      const int row = pos - (tile0 + tile * WARPS) * DECODE_BN;
#pragma unroll
      for (int i = 0; i < VW; ++i) {
        kt[row * ROW + lane * VW + i] = __float2bfloat16_rn(new_k[i]);
        kt[(DECODE_BN + row) * ROW + lane * VW + i] = __float2bfloat16_rn(new_v[i]);
      }
      __syncwarp();
    }
    attend_tile<DECODE_BN>(qf, kt, kt + DECODE_BN * ROW, (tile0 + tile * WARPS) * DECODE_BN, row_lo, row_hi,
                           sl2, m, l, o);
    __syncwarp();
    if (STAGES == 1) {  // the one stage is free again
      if (tile + 1 < tiles) load_tile(tile + 1, 0);
      cp_async_commit();
    } else if (FILLED) {
      if (tile + STAGES < tiles) load_tile(tile + STAGES, tile % STAGES);
      cp_async_commit();
    }
  }
  cp_async_wait<0>();
  OMNIA_TRACE_BLOCK(5);
  pdl_launch_dependents();  // the cache is read: the next kernel may begin its preamble

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  const int t = lane & 3;
  // The rows' states go to the block's partial: straight from the registers of a lone warp, or
  // (several warps) through shared memory, where warp 0 merges them, every lane its own dims.
  float* merge = reinterpret_cast<float*>(smem_raw);  // [WARPS][GROUP][D + 2]: accumulator, max (log2 units), sum
  if (WARPS > 1) __syncthreads();                     // every warp is done with its tiles
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = (lane >> 2) + 8 * r;
    if (row >= GROUP) continue;
    const size_t slot = (((size_t)blockIdx.z * nq + kvh * GROUP + row) * max_chunks + chunk);
    float* dst = WARPS == 1 ? part_o + slot * D : merge + ((size_t)warp * GROUP + row) * (D + 2);
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
      const int dim = 8 * j + 2 * t;
      if (dim >= D) continue;
      *reinterpret_cast<float2*>(dst + dim) = make_float2(o[j][2 * r], o[j][2 * r + 1]);
    }
    if (t == 0) {
      const float top = m[r] == -INFINITY ? -INFINITY : m[r] * sl2;  // the maximum in the exponent's units (log2)
      if (WARPS == 1) {
        part_ml[slot * 2] = top;
        part_ml[slot * 2 + 1] = l[r];
      } else {
        dst[D] = top;
        dst[D + 1] = l[r];
      }
    }
  }
  if (WARPS > 1) {
    __syncthreads();
    if (warp != 0) return;
    for (int row = 0; row < GROUP; ++row) {
      const size_t slot = (((size_t)blockIdx.z * nq + kvh * GROUP + row) * max_chunks + chunk);
      float top = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) top = fmaxf(top, merge[((size_t)w * GROUP + row) * (D + 2) + D]);
      float weight[WARPS], sum = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float* src = merge + ((size_t)w * GROUP + row) * (D + 2);
        weight[w] = src[D] == -INFINITY ? 0.f : exp2f(src[D] - top);
        sum += src[D + 1] * weight[w];
      }
      for (int dim = lane; dim < D; dim += 32) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) acc += merge[((size_t)w * GROUP + row) * (D + 2) + dim] * weight[w];
        part_o[slot * D + dim] = acc;
      }
      if (lane == 0) {
        part_ml[slot * 2] = top;
        part_ml[slot * 2 + 1] = sum;
      }
    }
  }
  // Whoever finishes last merges: publish the partial, take a ticket, and if it is the last
  // one of this (request, head group), read all partials back and write the output.
  __threadfence();
  __syncwarp();
  const int c0 = first / chunk_keys, c1 = pos / chunk_keys;
  int ticket = 0;
  int* counter = tickets + (size_t)blockIdx.z * nkv + kvh;
  if (lane == 0) ticket = atomicAdd(counter, 1);
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  OMNIA_TRACE_BLOCK(6);
  if (ticket != c1 - c0) return;
  if (lane == 0) *counter = 0;
  __threadfence();
  // Two heads at a time (their loads travel together; one at a time where a head's rows would not
  // fit in registers twice), then the odd one.
  constexpr int TOGETHER = D <= 128 ? 2 : 1;
  // The block's rings are idle by now: the least they hold, in floats, stages the chunks' accumulators.
  constexpr int STAGE_FLOATS = WARPS * STAGES * 2 * DECODE_BN * ROW * (int)sizeof(bf16) / (int)sizeof(float);
#pragma unroll 1
  for (int r = 0; r + TOGETHER <= GROUP; r += TOGETHER) {
    const int head = kvh * GROUP + r;
    combine_heads<TOGETHER>(part_o, part_ml, ((size_t)blockIdx.z * nq + head) * max_chunks, max_chunks, c0, c1,
                     gate ? gate + token * gate_stride + (size_t)head * D : nullptr, out + (token * nq + head) * D,
                     reinterpret_cast<float*>(smem_raw), STAGE_FLOATS);
  }
  if (GROUP % TOGETHER) {
    const int head = kvh * GROUP + GROUP - 1;
    combine_heads<1>(part_o, part_ml, ((size_t)blockIdx.z * nq + head) * max_chunks, max_chunks, c0, c1,
                     gate ? gate + token * gate_stride + (size_t)head * D : nullptr, out + (token * nq + head) * D,
                     reinterpret_cast<float*>(smem_raw), STAGE_FLOATS);
  }
  OMNIA_TRACE_BLOCK(7);
}

// ---------------------------------------------------------------------------------------

extern "C" int omnia_attention_tc_info(int* head_dim, int* group, int* tokens_per_block) {
  *head_dim = HEAD_DIM;
  *group = GROUP;
  *tokens_per_block = TOKENS_PER_BLOCK;
  return 0;
}

extern "C" int omnia_attention_prefill_tc(const void* q, const void* pages, const int* block_table,
                                          const int* cu_seqlens, const int* seq_lens,
                                          const int* work, int blocks, const void* gate,
                                          int gate_stride, void* out, int max_pages, int num_pages,
                                          int nq, int nkv, int page_size, int window, float scale,
                                          int* err, cudaStream_t stream) {
  if (blocks == 0) return 0;
  if (nq != nkv * GROUP) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)(BM + 4 * BN) * ROW * sizeof(bf16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  launch_pdl(attention_prefill_kernel, dim3(blocks, nkv), 128, smem, stream, 
      (const bf16*)q, (const bf16*)pages, block_table, cu_seqlens, seq_lens, work, (const bf16*)gate,
      gate_stride, (bf16*)out, max_pages, num_pages, nq, nkv, page_size, window, scale, err);
  return OMNIA_LAUNCH_RESULT();
}

// Shared memory of an SM, the most a block may ask for, and what a block costs beside its dynamic
// part (the system's kilobyte and the kernel's static arrays). Both decode entry points allow the
// kernels the same dynamic size, so neither undoes the other's setting.
constexpr size_t SM_SHARED = 228 * 1024, BLOCK_MOST = 227 * 1024, BLOCK_OVERHEAD = 1024 + 5 * 1024;

// proj non-null selects the fused mode: the kernel first does the step's QK-norm (eps < 0: none),
// rotation (inv_freq: head_dim / 2 inverse frequencies, or null) and cache write from the
// projected rows [tokens, stride] with q, k, v heads at q_col, k_col, v_col, and q is not read.
// It needs a head size that is a multiple of 32.
extern "C" int omnia_attention_decode_tc(const void* q, const void* pages, const int* block_table,
                                         const int* cu_seqlens, const int* seq_lens,
                                         const int* seq_ids, int requests, float* part_o,
                                         float* part_ml, int* tickets, int chunk_keys,
                                         int max_chunks, const void* gate, int gate_stride,
                                         void* out, int max_pages, int num_pages, int nq, int nkv,
                                         int page_size, int window, float scale, int warps,
                                         const void* proj, int proj_stride, int q_col, int k_col, int v_col,
                                         float eps, const float* inv_freq, const long long* slot_mapping,
                                         int spread, int* err, cudaStream_t stream) {
  if (requests == 0) return 0;
  if (requests < 0 || nkv < 1 || nq != nkv * GROUP || chunk_keys <= 0 || chunk_keys % DECODE_BN != 0 ||
      max_chunks < 1 || max_pages < 1 || num_pages < 1 || page_size < 1 || (warps != 1 && warps != 4))
    return (int)cudaErrorInvalidValue;
  if (proj != nullptr && (D % 32 != 0 || slot_mapping == nullptr || proj_stride % 2 || q_col % 2 || k_col % 2 || v_col % 2))
    return (int)cudaErrorInvalidValue;
  const FusedQK fused{(const bf16*)proj, proj_stride, q_col, k_col, v_col, eps, inv_freq, slot_mapping,
                      (bf16*)const_cast<void*>(pages), (long long)num_pages * page_size};
  // One warp: a two-stage ring. Four warps: one stage each (a warp has few tiles), and the merge area
  // fits in it; where the grid is at most a block per SM, two stages each: a warp's tiles are then
  // all on their way before it needs the first (a single request of 4,096 tokens: each warp has two).
  const int sms = omnia_sm_count();
  const bool deep = warps == 4 && (long long)max_chunks * nkv * requests <= sms &&
                    (size_t)(8 * 2 * DECODE_BN) * ROW * sizeof(bf16) <= BLOCK_MOST - BLOCK_OVERHEAD;  // (head size 256: too large)
  size_t smem = (size_t)((warps == 1 ? DECODE_STAGES : deep ? 8 : 4) * 2 * DECODE_BN) * ROW * sizeof(bf16);
  static bool configured[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  if (!configured[device]) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<1, DECODE_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(BLOCK_MOST - BLOCK_OVERHEAD));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_decode_kernel<4, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)(BLOCK_MOST - BLOCK_OVERHEAD));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_decode_kernel<4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)(BLOCK_MOST - BLOCK_OVERHEAD));
    if (e != cudaSuccess) return (int)e;
    configured[device] = true;
  }
  if (spread) {
    // The blocks are handed to SMs as these become free, as many to an SM as fit, and the kernel
    // before this one frees its SMs one after the other: left alone, six blocks each go to the first
    // SMs (seen: 512 blocks on 86 of 148 SMs) and the rest of the GPU idles. So every block asks
    // for so much shared memory that an SM holds no more than its share of the grid.
    const long long blocks = (long long)max_chunks * nkv * requests;
    const long long share = (blocks + sms - 1) / sms;
    const size_t room = SM_SHARED / (size_t)share;
    if (room > smem + BLOCK_OVERHEAD) smem = (room > BLOCK_MOST ? BLOCK_MOST : room) - BLOCK_OVERHEAD;
  }
  if (warps == 1)
    launch_pdl(attention_decode_kernel<1, DECODE_STAGES>, dim3(max_chunks, nkv, requests), 32, smem, stream,
        (const bf16*)q, (const bf16*)pages, block_table, cu_seqlens, seq_lens, seq_ids, part_o, part_ml,
        tickets, (const bf16*)gate, gate_stride, (bf16*)out, chunk_keys, max_chunks, max_pages,
        num_pages, nq, nkv, page_size, window, scale, fused, err);
  else if (deep)
    launch_pdl(attention_decode_kernel<4, 2>, dim3(max_chunks, nkv, requests), 128, smem, stream,
        (const bf16*)q, (const bf16*)pages, block_table, cu_seqlens, seq_lens, seq_ids, part_o, part_ml,
        tickets, (const bf16*)gate, gate_stride, (bf16*)out, chunk_keys, max_chunks, max_pages,
        num_pages, nq, nkv, page_size, window, scale, fused, err);
  else
    launch_pdl(attention_decode_kernel<4, 1>, dim3(max_chunks, nkv, requests), 128, smem, stream,
        (const bf16*)q, (const bf16*)pages, block_table, cu_seqlens, seq_lens, seq_ids, part_o, part_ml,
        tickets, (const bf16*)gate, gate_stride, (bf16*)out, chunk_keys, max_chunks, max_pages,
        num_pages, nq, nkv, page_size, window, scale, fused, err);
  return OMNIA_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------------
// The decode kernel for callers that cannot allocate (see attention_static.h): the three
// scratch buffers are carved out of one array in the library's device image.
#include "attention_static.h"

#include <stdio.h>

#include <mutex>

static __device__ __align__(256) unsigned char static_scratch[OMNIA_STATIC_SCRATCH_BYTES];

static thread_local char static_error[256] = "";

extern "C" const char* omnia_attention_static_error(void) { return static_error; }

extern "C" int omnia_attention_decode_tc_static(const void* q, const void* pages,
                                                const int* block_table, const int* cu_seqlens,
                                                const int* seq_lens, const int* seq_ids,
                                                int requests, int chunk_keys, int max_chunks,
                                                const void* gate, int gate_stride, void* out,
                                                int max_pages, int num_pages, int nq, int nkv,
                                                int page_size, int window, float scale, int* err,
                                                cudaStream_t stream) {
  static_error[0] = 0;
  if (requests == 0) return 0;
  if (requests < 0 || nkv < 1 || max_chunks < 1 || max_pages < 1 || num_pages < 1 || page_size < 1) {
    snprintf(static_error, sizeof static_error,
             "requests (%d) must not be negative; nkv (%d), max_chunks (%d), max_pages (%d), num_pages (%d) "
             "and page_size (%d) must be at least 1", requests, nkv, max_chunks, max_pages, num_pages, page_size);
    return (int)cudaErrorInvalidValue;
  }
  if (nq != nkv * GROUP || chunk_keys <= 0 || chunk_keys % DECODE_BN != 0) {
    snprintf(static_error, sizeof static_error,
             "this library is compiled for %d query heads per key/value head and chunks that are a "
             "positive multiple of %d keys (given: nq %d, nkv %d, chunk_keys %d)", GROUP, DECODE_BN, nq, nkv,
             chunk_keys);
    return (int)cudaErrorInvalidValue;
  }
  const long long slots = (long long)requests * nq * max_chunks;
  const long long floats = slots * (D + 2), tickets = (long long)requests * nkv;
  if (floats > OMNIA_STATIC_SCRATCH_FLOATS || tickets > OMNIA_STATIC_TICKETS) {
    snprintf(static_error, sizeof static_error,
             "the call needs %lld scratch floats and %lld tickets; the static scratch holds %d and %d "
             "(requests * nq * max_chunks * (head_dim + 2) floats, requests * nkv tickets)",
             floats, tickets, OMNIA_STATIC_SCRATCH_FLOATS, OMNIA_STATIC_TICKETS);
    return OMNIA_STATIC_TOO_LARGE;
  }
  // Once per device, with that device current: the array's name is only a host-side handle;
  // the kernel needs the address the symbol has on this device.
  constexpr int MAX_DEVICES = 64;
  static unsigned char* device_address[MAX_DEVICES] = {nullptr};
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= MAX_DEVICES) {
    snprintf(static_error, sizeof static_error, "cudaGetDevice failed or device %d is beyond %d", device,
             MAX_DEVICES);
    return e != cudaSuccess ? (int)e : OMNIA_STATIC_NO_DEVICE;
  }
  {
  static std::mutex setup;  // two host threads may make a device's first call at once
  std::lock_guard<std::mutex> held(setup);
  if (device_address[device] == nullptr) {
    unsigned char* address = nullptr;
    e = cudaGetSymbolAddress((void**)&address, static_scratch);
    if (e != cudaSuccess) {
      snprintf(static_error, sizeof static_error, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return (int)e;
    }
    e = cudaFuncSetAttribute(attention_decode_kernel<1, DECODE_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(BLOCK_MOST - BLOCK_OVERHEAD));
    if (e != cudaSuccess) {
      snprintf(static_error, sizeof static_error, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return (int)e;
    }
    device_address[device] = address;
  }
  }
  float* part_o = reinterpret_cast<float*>(device_address[device]);
  float* part_ml = part_o + slots * D;
  int* ticket_area = reinterpret_cast<int*>(device_address[device] + (size_t)OMNIA_STATIC_SCRATCH_FLOATS * 4);
  // The tickets must start at zero, whatever an earlier call left behind.
  e = cudaMemsetAsync(ticket_area, 0, (size_t)tickets * sizeof(int), stream);
  if (e != cudaSuccess) {
    snprintf(static_error, sizeof static_error, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    return (int)e;
  }
  const size_t smem = (size_t)(DECODE_STAGES * 2 * DECODE_BN) * ROW * sizeof(bf16);
  launch_pdl(attention_decode_kernel<1, DECODE_STAGES>, dim3(max_chunks, nkv, requests), 32, smem, stream,
      (const bf16*)q, (const bf16*)pages, block_table, cu_seqlens, seq_lens, seq_ids, part_o, part_ml,
      ticket_area, (const bf16*)gate, gate_stride, (bf16*)out, chunk_keys, max_chunks, max_pages,
      num_pages, nq, nkv, page_size, window, scale, FusedQK{}, err);
  e = cudaGetLastError();
  if (e != cudaSuccess) snprintf(static_error, sizeof static_error, "launch: %s", cudaGetErrorString(e));
  return (int)e;
}
