// Next-token choice on the GPU, a cluster of eight blocks per row of float32 logits.
//
// Order of the stages, as the reference composes them (repetition penalty on the raw
// logits, then temperature -> top_k -> top_p -> min_p, then a categorical draw):
//   penalty:     each id seen in the recent history: logit > 0 ? logit / v : logit * v
//   temperature: s = logit / t        (t == 0 selects greedy: the first largest logit)
//   top_k:       keep s >= (k-th largest s); a tie at the k-th value keeps the whole tie
//   top_p:       with e = exp(s - max) over what is kept and Z = sum e: keep e >= c where c
//                is the smallest value whose strictly-greater mass is below p * Z
//   min_p:       keep e >= p   (the most probable token has e == 1)
//   draw:        argmax of s + Gumbel noise from Philox4x32-10(seed; draw index, token id)
// Thresholds are found by radix selection on the bit patterns of the floats (see sample_kernel).
#include <cooperative_groups.h>

#include "common.cuh"

#define SAMPLE_THREADS 512
#define SAMPLE_CLUSTER 8

__device__ __forceinline__ unsigned int order_key(float v) {
  // Monotone map float -> uint: larger float, larger key.
  const unsigned int b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ void philox4x32_10(unsigned int c0, unsigned int c1, unsigned int c2,
                                              unsigned int c3, unsigned int k0, unsigned int k1,
                                              unsigned int* out) {
  const unsigned int M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned int hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const unsigned int hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    const unsigned int n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

struct ArgMax {
  float v;
  int i;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  // Larger value wins; on a tie the lower index does.
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax a, ArgMax* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = a;
  __syncthreads();
  if (warp == 0) {
    const int warps = blockDim.x >> 5;
    ArgMax t = lane < warps ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax b;
      b.v = __shfl_xor_sync(0xffffffffu, t.v, o);
      b.i = __shfl_xor_sync(0xffffffffu, t.i, o);
      t = better(t, b);
    }
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// A row is shared by a cluster of SAMPLE_CLUSTER blocks, each holding one slice of the row's
// scaled logits in shared memory. Thresholds are found by radix selection on the bit patterns of
// the floats (monotone for the values compared), eight bits a pass: every block builds a histogram
// of its slice, the histograms are added across the cluster through distributed shared memory,
// and every block walks the sum from the top to the bin that holds the threshold. Counts are
// integers and probability mass is added in fixed point (2^-40), so the sums do not depend on
// their order and a seeded run repeats bit for bit.
struct SampleShared {
  unsigned int count[256];           // this block's histogram of the pass
  unsigned int limb[3][256];         // its mass in three limbs of 16 bits (32-bit atomics; at most 2^15 additions)
  unsigned int total_count[2][256];  // the cluster's, of alternate passes: every block adds into every block's
  unsigned int total_limb[2][3][256];  // the cluster's mass in three limbs of 20 bits (32-bit remote atomics)
  ArgMax first_best, draw_best;      // this block's candidates, read by the whole cluster
  ArgMax ascratch[33];
  unsigned int digit;                // the bin a pass settled on
  unsigned long long above;          // count or mass of the bins above it
  unsigned long long limit;          // what the count or mass above an element must stay below
};

__device__ __forceinline__ unsigned long long fixed_mass(float e) { return __float2ull_rn(e * 1099511627776.f); }

// One histogram pass over this block's slice. `item(j, key, weight)` gives element j's 32-bit key
// and fixed-point mass and says whether the element takes part at all; of those, only elements
// whose key matches `prefix` in the bits above `shift + 8` are counted (all, when shift is 24).
// A lane adds up consecutive elements of one bin in registers (in the upper digits nearly all
// elements share a bin) and goes to shared memory when the bin changes and at the end, where
// the lanes of a warp that hold the same bin are added up first.
template <bool MASS, typename Item>
__device__ __forceinline__ void histogram_pass(SampleShared& sh, int buf, int n, unsigned int prefix, int shift,
                                               Item item) {
  for (int b = threadIdx.x; b < 256; b += blockDim.x) {
    sh.count[b] = 0u;
    sh.limb[0][b] = sh.limb[1][b] = sh.limb[2][b] = 0u;
    sh.total_count[buf ^ 1][b] = 0u;  // the next pass's totals: nobody adds to them before this pass's barrier
    sh.total_limb[buf ^ 1][0][b] = sh.total_limb[buf ^ 1][1][b] = sh.total_limb[buf ^ 1][2][b] = 0u;
  }
  __syncthreads();
  unsigned int held = 256u, held_count = 0u;  // 256: nothing held yet
  unsigned long long held_mass = 0ull;
  // A lane's mass is below 2^47 (fewer than 2^6 elements of less than 2^41 each).
  auto flush = [&](unsigned int bin, unsigned int count, unsigned long long mass) {
    atomicAdd(&sh.count[bin], count);
    if (MASS) {
      atomicAdd(&sh.limb[0][bin], (unsigned int)(mass & 0xFFFFu));
      atomicAdd(&sh.limb[1][bin], (unsigned int)((mass >> 16) & 0xFFFFu));
      atomicAdd(&sh.limb[2][bin], (unsigned int)(mass >> 32));
    }
  };
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    unsigned int key = 0u;
    unsigned long long weight = 0ull;
    if (!item(j, key, weight)) continue;
    if (shift < 24 && (key >> (shift + 8)) != (prefix >> (shift + 8))) continue;
    const unsigned int digit = (key >> shift) & 255u;
    if (digit != held) {
      if (held_count) flush(held, held_count, held_mass);
      held = digit;
      held_count = 0u;
      held_mass = 0ull;
    }
    ++held_count;
    held_mass += weight;
  }
  // What the lanes still hold. When all of a warp's lanes that hold something hold the same bin
  // (the usual case in the upper digits), they are added up first and one lane goes to shared memory.
  const unsigned int holders = __ballot_sync(0xffffffffu, held_count != 0u);
  if (holders == 0u) return;
  const unsigned int reference = __shfl_sync(0xffffffffu, held, __ffs(holders) - 1);
  if (__all_sync(0xffffffffu, held_count == 0u || held == reference)) {
    const unsigned int count = __reduce_add_sync(0xffffffffu, held_count);
    unsigned long long mass = 0ull;
    if (MASS) {  // 32 lanes' 16-bit pieces add up to less than 2^21
      const unsigned int p0 = __reduce_add_sync(0xffffffffu, (unsigned int)(held_mass & 0xFFFFu));
      const unsigned int p1 = __reduce_add_sync(0xffffffffu, (unsigned int)((held_mass >> 16) & 0xFFFFu));
      const unsigned int p2 = __reduce_add_sync(0xffffffffu, (unsigned int)(held_mass >> 32));
      mass = (unsigned long long)p0 + ((unsigned long long)p1 << 16) + ((unsigned long long)p2 << 32);
    }
    if ((threadIdx.x & 31) == 0) {
      atomicAdd(&sh.count[reference], count);
      if (MASS) {  // a warp's mass is below 2^52: the top limb takes what is above 32 bits
        atomicAdd(&sh.limb[0][reference], (unsigned int)(mass & 0xFFFFu));
        atomicAdd(&sh.limb[1][reference], (unsigned int)((mass >> 16) & 0xFFFFu));
        atomicAdd(&sh.limb[2][reference], (unsigned int)(mass >> 32));
      }
    }
  } else if (held_count) {
    flush(held, held_count, held_mass);
  }
}

// Adds this block's histogram into every block's totals of buffer `buf` (remote atomics, nobody
// waits for them), then the cluster meets: after that each block reads the sums in its own
// shared memory.
__device__ __forceinline__ void cluster_totals(cooperative_groups::cluster_group& cluster, SampleShared& sh, int buf,
                                               bool mass) {
  __syncthreads();
  for (int b = threadIdx.x; b < 256; b += blockDim.x) {
    const unsigned int c = sh.count[b];
    if (c == 0u) continue;
    const unsigned long long m = (unsigned long long)sh.limb[0][b] + ((unsigned long long)sh.limb[1][b] << 16) +
                                 ((unsigned long long)sh.limb[2][b] << 32);
#pragma unroll
    for (unsigned int r = 0; r < SAMPLE_CLUSTER; ++r) {
      SampleShared* other = cluster.map_shared_rank(&sh, r);
      atomicAdd(&other->total_count[buf][b], c);
      if (mass && m) {  // a block's mass of a bin is below 2^58; eight blocks' limbs stay below 2^23
        atomicAdd(&other->total_limb[buf][0][b], (unsigned int)(m & 0xFFFFFu));
        atomicAdd(&other->total_limb[buf][1][b], (unsigned int)((m >> 20) & 0xFFFFFu));
        atomicAdd(&other->total_limb[buf][2][b], (unsigned int)(m >> 40));
      }
    }
  }
  cluster.sync();
}

// Warp 0 walks the cluster's histogram from the top, lane l taking bins 255 - 8 l down to 248 - 8 l:
// the lowest bin that holds an element with less than `limit` (counts, or mass) in the bins above
// it. With `fraction` >= 0 the limit is first set to that fraction of the histogram's whole mass,
// rounded up (an integer is below p * Z exactly when it is below the next integer at or above it).
// Leaves the bin, what lies above it, and the limit in shared memory.
__device__ __forceinline__ void select_bin(SampleShared& sh, int buf, bool by_mass, unsigned long long limit,
                                           float fraction) {
  const int lane = threadIdx.x;
  unsigned long long w[8], sum = 0ull;
  unsigned int c[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int b = 255 - 8 * lane - i;
    c[i] = sh.total_count[buf][b];
    w[i] = by_mass ? (unsigned long long)sh.total_limb[buf][0][b] + ((unsigned long long)sh.total_limb[buf][1][b] << 20) +
                         ((unsigned long long)sh.total_limb[buf][2][b] << 40)
                   : (unsigned long long)c[i];
    sum += w[i];
  }
  unsigned long long inclusive = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long up = __shfl_up_sync(0xffffffffu, inclusive, o);
    if (lane >= o) inclusive += up;
  }
  if (fraction >= 0.f) {
    const unsigned long long all = __shfl_sync(0xffffffffu, inclusive, 31);
    limit = (unsigned long long)ceil((double)fraction * (double)all);
  }
  unsigned long long above = inclusive - sum, chosen_above = 0ull;
  int chosen = -1;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (c[i] != 0u && above < limit) {
      chosen = 255 - 8 * lane - i;
      chosen_above = above;
    }
    above += w[i];
  }
  const unsigned int has = __ballot_sync(0xffffffffu, chosen >= 0);
  const int from = has ? 31 - __clz(has) : 0;  // the lane with the lowest such bin
  chosen = __shfl_sync(0xffffffffu, chosen, from);
  chosen_above = __shfl_sync(0xffffffffu, chosen_above, from);
  if (lane == 0) {
    sh.digit = has ? (unsigned int)chosen : 0u;
    sh.above = has ? chosen_above : 0ull;
    sh.limit = limit;
  }
}

__global__ void __cluster_dims__(SAMPLE_CLUSTER, 1, 1) __launch_bounds__(SAMPLE_THREADS, 2)
sample_kernel(float* __restrict__ logits, long long stride, int vocab, int slice, int cached,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ penalty, const int* __restrict__ history, int history_len,
              const long long* __restrict__ seeds, const long long* __restrict__ draws,
              int* __restrict__ out) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float sv[];  // this block's slice of s = logit / temperature, when it fits
  __shared__ SampleShared sh;
  const int row = blockIdx.x / SAMPLE_CLUSTER, rank = (int)cluster.block_rank();
  float* z = logits + (size_t)row * stride;
  const int begin = min(vocab, rank * slice), n = min(vocab, begin + slice) - begin;

  // Repetition penalty: once per distinct recent id, on the raw logit, by the block whose slice holds it.
  const float pen = penalty ? penalty[row] : 1.f;
  if (pen != 1.f && history != nullptr) {
    const int* hist = history + (size_t)row * history_len;
    if ((int)threadIdx.x < history_len) {
      const int id = hist[threadIdx.x];
      bool first = id >= begin && id < begin + n;
      for (int j = 0; first && j < (int)threadIdx.x; ++j) first = hist[j] != id;
      if (first) z[id] = z[id] > 0.f ? z[id] / pen : z[id] * pen;
    }
    __syncthreads();
  }

  // The largest raw logit (the greedy choice, and the softmax's maximum), first index on a tie.
  const float temp = temperature ? temperature[row] : 0.f;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float v = z[begin + j];
    best = better(best, ArgMax{v, begin + j});
    if (cached) sv[j] = temp > 0.f ? v / temp : v;
  }
  best = block_argmax(best, sh.ascratch);
  if (threadIdx.x == 0) sh.first_best = best;
  for (int b = threadIdx.x; b < 256; b += blockDim.x) {  // the first pass's totals start at zero
    sh.total_count[0][b] = 0u;
    sh.total_limb[0][0][b] = sh.total_limb[0][1][b] = sh.total_limb[0][2][b] = 0u;
  }
  cluster.sync();
  for (unsigned int r = 0; r < cluster.num_blocks(); ++r) best = better(best, cluster.map_shared_rank(&sh, r)->first_best);
  if (temp <= 0.f) {
    if (rank == 0 && threadIdx.x == 0) out[row] = best.i;
    cluster.sync();  // nobody leaves while its shared memory may still be read
    return;
  }
  const float smax = best.v / temp;
  auto s_of = [&](int j) { return cached ? sv[j] : z[begin + j] / temp; };
  int buf = 0;

  // top_k: the k-th largest key (a tie at it is kept whole).
  unsigned int kkey = 0u;  // keeps everything
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < vocab) {
    unsigned long long want = (unsigned long long)k;  // the rank looked for among the elements that match the prefix
    for (int shift = 24; shift >= 0; shift -= 8, buf ^= 1) {
      histogram_pass<false>(sh, buf, n, kkey, shift, [&](int j, unsigned int& key, unsigned long long&) {
        key = order_key(s_of(j));
        return true;
      });
      cluster_totals(cluster, sh, buf, false);
      if (threadIdx.x < 32) select_bin(sh, buf, false, want, -1.f);  // the k-th largest has fewer than k above it
      __syncthreads();
      kkey |= sh.digit << shift;
      want -= sh.above;
      __syncthreads();
    }
  }

  // top_p over what top_k kept: with e = exp(s - max) and Z its sum, the smallest e whose
  // strictly greater mass is below p * Z. min_p: e >= p (the most probable token has e == 1).
  float ecut = 0.f;
  const float p = top_p ? top_p[row] : 1.f;
  if (p < 1.f) {
    unsigned int ckey = 0u;
    unsigned long long limit = 0ull;
    for (int shift = 24; shift >= 0; shift -= 8, buf ^= 1) {
      histogram_pass<true>(sh, buf, n, ckey, shift, [&](int j, unsigned int& key, unsigned long long& weight) {
        const float s = s_of(j);
        if (order_key(s) < kkey) return false;  // not kept by top_k
        const float e = expf(s - smax);
        key = __float_as_uint(e);  // e >= 0: its bits order it
        weight = fixed_mass(e);
        return true;
      });
      cluster_totals(cluster, sh, buf, true);
      // The lowest bin that holds an element whose strictly greater mass is below p * Z: a bin's
      // largest element has exactly the mass of the bins above it.
      if (threadIdx.x < 32) select_bin(sh, buf, true, limit, shift == 24 ? p : -1.f);
      __syncthreads();
      ckey |= sh.digit << shift;
      limit = sh.limit - sh.above;
      __syncthreads();
    }
    ecut = __uint_as_float(ckey);
  }
  const float mp = min_p ? min_p[row] : 0.f;
  if (mp > ecut) ecut = mp;

  // The draw: Gumbel-max over the kept tokens.
  const unsigned long long seed = (unsigned long long)seeds[row];
  const unsigned long long draw = (unsigned long long)draws[row];
  ArgMax pick{-INFINITY, 0x7fffffff};
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float s = s_of(j);
    if (order_key(s) < kkey) continue;
    if (expf(s - smax) < ecut) continue;
    unsigned int r[4];
    philox4x32_10((unsigned int)(begin + j), 0u, (unsigned int)draw, (unsigned int)(draw >> 32),
                  (unsigned int)seed, (unsigned int)(seed >> 32), r);
    const float u = ((float)(r[0] >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float g = -logf(-logf(u));
    pick = better(pick, ArgMax{s + g, begin + j});
  }
  pick = block_argmax(pick, sh.ascratch);
  if (threadIdx.x == 0) sh.draw_best = pick;
  cluster.sync();
  if (rank == 0 && threadIdx.x == 0) {
    for (unsigned int r = 1; r < cluster.num_blocks(); ++r) pick = better(pick, cluster.map_shared_rank(&sh, r)->draw_best);
    out[row] = pick.i;
  }
  cluster.sync();  // nobody leaves while its shared memory may still be read
}

// Greedy choice for many rows at once: stage 1 finds the best of each of ARGMAX_PARTS slices
// of a row, stage 2 the best of those (ties go to the lower index in both).
#define ARGMAX_PARTS 32

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, long long stride, int vocab,
                      float* __restrict__ part_v, int* __restrict__ part_i) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ ArgMax ascratch[33];
  const int row = blockIdx.y, part = blockIdx.x;
  const float* z = logits + (size_t)row * stride;
  const int per = (vocab + ARGMAX_PARTS - 1) / ARGMAX_PARTS;
  const int begin = part * per, end = min(vocab, begin + per);
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) best = better(best, ArgMax{z[i], i});
  best = block_argmax(best, ascratch);
  if (threadIdx.x == 0) {
    part_v[row * ARGMAX_PARTS + part] = best.v;
    part_i[row * ARGMAX_PARTS + part] = best.i;
  }
}

__global__ void __launch_bounds__(32)
argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                    int* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x, lane = threadIdx.x;
  ArgMax a{part_v[row * ARGMAX_PARTS + lane], part_i[row * ARGMAX_PARTS + lane]};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  if (lane == 0) out[row] = a.i;
}

// part_v, part_i: scratch of rows * 32 elements each.
extern "C" int omnia_argmax(const float* logits, long long stride, int rows, int vocab,
                            float* part_v, int* part_i, int* out, cudaStream_t stream) {
  if (rows == 0) return 0;
  launch_pdl(argmax_partial_kernel, dim3(ARGMAX_PARTS, rows), 256, 0, stream, logits, stride, vocab, part_v,
                                                                     part_i);
  launch_pdl(argmax_final_kernel, rows, 32, 0, stream, part_v, part_i, out);
  return OMNIA_LAUNCH_RESULT();
}

extern "C" int omnia_sample(float* logits, long long stride, int rows, int vocab,
                            const float* temperature, const int* top_k, const float* top_p,
                            const float* min_p, const float* penalty, const int* history,
                            int history_len, const long long* seeds, const long long* draws,
                            int* out, cudaStream_t stream) {
  if (rows == 0) return 0;
  // History entries are handled one per thread; the histograms' limbs hold up to 2^16 logits a block.
  if (history_len > SAMPLE_THREADS || vocab > SAMPLE_CLUSTER * 65536) return (int)cudaErrorInvalidValue;
  // A block keeps its slice of the row in shared memory when it fits (up to 8 x 49,152 logits a row);
  // beyond that the slices are read from the logits again in every pass.
  const int slice = (vocab + SAMPLE_CLUSTER - 1) / SAMPLE_CLUSTER;
  const int cached = slice <= 49152 ? 1 : 0;
  const size_t smem = cached ? (size_t)slice * sizeof(float) : 0;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  launch_pdl(sample_kernel, rows * SAMPLE_CLUSTER, SAMPLE_THREADS, smem, stream, logits, stride, vocab, slice, cached,
             temperature, top_k, top_p, min_p, penalty, history, history_len, seeds, draws, out);
  return OMNIA_LAUNCH_RESULT();
}
