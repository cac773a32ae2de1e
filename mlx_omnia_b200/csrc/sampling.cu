// Next-token choice on the GPU, one block per row of float32 logits.
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
// Thresholds are found by bisection on the bit patterns of the floats (monotone for the
// values compared), each probe being one block-wide reduction in a fixed order, so a
// seeded run repeats bit for bit.
#include "common.cuh"

#define SAMPLE_THREADS 1024

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

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(float* __restrict__ logits, long long stride, int vocab,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ penalty, const int* __restrict__ history, int history_len,
              const long long* __restrict__ seeds, const long long* __restrict__ draws,
              int* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float fscratch[33];
  __shared__ ArgMax ascratch[33];
  const int row = blockIdx.x;
  float* z = logits + (size_t)row * stride;

  // Repetition penalty: once per distinct recent id, on the raw logit.
  const float pen = penalty ? penalty[row] : 1.f;
  if (pen != 1.f && history != nullptr) {
    const int* hist = history + (size_t)row * history_len;
    if ((int)threadIdx.x < history_len) {
      const int id = hist[threadIdx.x];
      bool first = id >= 0 && id < vocab;
      for (int j = 0; first && j < (int)threadIdx.x; ++j) first = hist[j] != id;
      if (first) z[id] = z[id] > 0.f ? z[id] / pen : z[id] * pen;
    }
    __syncthreads();
  }

  const float temp = temperature ? temperature[row] : 0.f;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgMax{z[i], i});
  best = block_argmax(best, ascratch);
  if (temp <= 0.f) {
    if (threadIdx.x == 0) out[row] = best.i;
    return;
  }
  const float smax = best.v / temp;

  // top_k: the largest key u with count(key >= u) >= k.
  unsigned int kkey = 0u;  // keeps everything
  const int k = top_k ? top_k[row] : 0;
  if (k > 0 && k < vocab) {
    unsigned int u = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned int cand = u | (1u << bit);
      float cnt = 0.f;  // counts are exact in float32 up to 2^24 entries
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) cnt += order_key(z[i] / temp) >= cand;
      if (block_sum(cnt, fscratch) >= (float)k) u = cand;
    }
    kkey = u;
  }

  // Normaliser over what top_k kept.
  float zsum = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float s = z[i] / temp;
    if (order_key(s) >= kkey) zsum += expf(s - smax);
  }
  zsum = block_sum(zsum, fscratch);

  // top_p: the smallest threshold c (as a bit pattern of e > 0) with mass(e > c) < p * Z.
  float ecut = 0.f;
  const float p = top_p ? top_p[row] : 1.f;
  if (p < 1.f) {
    const float target = p * zsum;
    // f(c) = [mass(e > c) < target] is false for small c and true for large c; every e is
    // <= 1 and f(1.0f) is true (nothing lies above the maximum). Binary search over the bit
    // patterns of the non-negative floats for the smallest c with f(c) true.
    unsigned int lo = 0u, c = 0x3F800000u;
    while (lo < c) {
      const unsigned int mid = lo + ((c - lo) >> 1);
      const float cv = __uint_as_float(mid);
      float mass = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float s = z[i] / temp;
        if (order_key(s) >= kkey) {
          const float e = expf(s - smax);
          if (e > cv) mass += e;
        }
      }
      mass = block_sum(mass, fscratch);
      if (mass < target) c = mid; else lo = mid + 1u;
    }
    ecut = __uint_as_float(c);
  }
  const float mp = min_p ? min_p[row] : 0.f;
  if (mp > ecut) ecut = mp;

  // The draw: Gumbel-max over the kept tokens.
  const unsigned long long seed = (unsigned long long)seeds[row];
  const unsigned long long draw = (unsigned long long)draws[row];
  ArgMax pick{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float s = z[i] / temp;
    if (order_key(s) < kkey) continue;
    if (expf(s - smax) < ecut) continue;
    unsigned int r[4];
    philox4x32_10((unsigned int)i, 0u, (unsigned int)draw, (unsigned int)(draw >> 32),
                  (unsigned int)seed, (unsigned int)(seed >> 32), r);
    const float u = ((float)(r[0] >> 8) + 0.5f) * (1.0f / 16777216.0f);
    const float g = -logf(-logf(u));
    pick = better(pick, ArgMax{s + g, i});
  }
  pick = block_argmax(pick, ascratch);
  if (threadIdx.x == 0) out[row] = pick.i;
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
  if (history_len > SAMPLE_THREADS) return (int)cudaErrorInvalidValue;
  launch_pdl(sample_kernel, rows, SAMPLE_THREADS, 0, stream, logits, stride, vocab, temperature, top_k,
                                                     top_p, min_p, penalty, history, history_len,
                                                     seeds, draws, out);
  return OMNIA_LAUNCH_RESULT();
}
