// Embedding, norms, rotation + cache write, gated activation, logit cap, row gather.
// One row (token) per block unless said otherwise; float32 arithmetic throughout.
#include "common.cuh"

// ---------------------------------------------------------------------------------
// Embedding lookup with an optional weightless RMS norm: x[t] = rms0(table[ids[t]]).
// The residual stream x is float32 in both precisions.
template <typename T>
__global__ void embed_rmsnorm_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                     float* __restrict__ x, int hidden, int vocab, float eps,
                                     int normed, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(err, OMNIA_ERR_TOKEN_ID);
    id = 0;
  }
  const T* row = table + (size_t)id * hidden;
  float* out = x + (size_t)t * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = to_f32(row[i]);
    ss += v * v;
  }
  float scale = 1.f;
  if (normed) scale = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_f32(row[i]) * scale;
}

extern "C" int omnia_embed_rmsnorm(const int* ids, const void* table, float* x, int tokens,
                                   int hidden, int vocab, float eps, int normed, int dtype,
                                   int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(embed_rmsnorm_kernel<T>, tokens, 256, 0, stream, 
                                  ids, (const T*)table, x, hidden, vocab, eps, normed, err)));
  return OMNIA_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------
// h = x * rsqrt(mean(x^2) + eps) * w   (w may be null: weightless). x is float32.
template <typename T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               T* __restrict__ h, int hidden, float eps) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float scratch[33];
  const float* row = x + (size_t)blockIdx.x * hidden;
  T* out = h + (size_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) ss += row[i] * row[i];
  const float scale = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = row[i] * scale;
    if (w) v *= w[i];
    out[i] = from_f32<T>(v);
  }
}

extern "C" int omnia_rmsnorm(const float* x, const float* w, void* h, int rows, int hidden,
                             float eps, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  OMNIA_DISPATCH_DTYPE(dtype,
                       (launch_pdl(rmsnorm_kernel<T>, rows, 256, 0, stream, x, w, (T*)h, hidden, eps)));
  return OMNIA_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------
// The residual step of a block, in one pass over the row:
//   a  = branch                      (optionally normed: a * rsqrt(mean a^2 + eps_b) * wb)
//   x += a                           (float32, in place)
//   h  = x * rsqrt(mean x^2 + eps_o) * wo   (optional; wo may be null)
// The row is staged in shared memory as float32, so the branch is read once and x is
// read and written once.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ branch,
                                   const float* __restrict__ wb, float eps_b, int norm_branch,
                                   const float* __restrict__ wo, float eps_o, int norm_out,
                                   T* __restrict__ h, int hidden) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float row[];
  __shared__ float scratch[33];
  float* xr = x + (size_t)blockIdx.x * hidden;
  const T* br = branch + (size_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float a = to_f32(br[i]);
    row[i] = a;
    ss += a * a;
  }
  float scale_b = 1.f;
  if (norm_branch) scale_b = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps_b);
  ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float a = row[i];
    if (norm_branch) {
      a *= scale_b;
      if (wb) a *= wb[i];
    }
    const float v = xr[i] + a;
    xr[i] = v;
    row[i] = v;
    ss += v * v;
  }
  if (!norm_out) return;
  const float scale_o = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps_o);
  T* out = h + (size_t)blockIdx.x * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = row[i] * scale_o;
    if (wo) v *= wo[i];
    out[i] = from_f32<T>(v);
  }
}

// The same residual step with the whole row in registers: every load of the row (branch, x
// and both weights) is issued before the first reduction, so a row costs one memory round
// trip instead of three. hidden % 4 == 0 and hidden <= 4 * ITERS * blockDim.
template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<unsigned*>(&a);
    t.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
  }
};

template <typename T, int ITERS>
__global__ void add_rmsnorm_reg_kernel(float* __restrict__ x, const T* __restrict__ branch,
                                       const float* __restrict__ wb, float eps_b, int norm_branch,
                                       const float* __restrict__ wo, float eps_o, int norm_out,
                                       T* __restrict__ h, int hidden) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float scratch[33];
  float* xr = x + (size_t)blockIdx.x * hidden;
  const T* br = branch + (size_t)blockIdx.x * hidden;
  float a[ITERS][4], xv[ITERS][4], gb[ITERS][4], go[ITERS][4];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    const bool live = i < hidden;
#pragma unroll
    for (int k = 0; k < 4; ++k) a[it][k] = xv[it][k] = 0.f, gb[it][k] = go[it][k] = 1.f;
    if (live) {
      Vec4<T>::load(br + i, a[it]);
      Vec4<float>::load(xr + i, xv[it]);
      if (norm_branch && wb) Vec4<float>::load(wb + i, gb[it]);
      if (norm_out && wo) Vec4<float>::load(wo + i, go[it]);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it)
#pragma unroll
    for (int k = 0; k < 4; ++k) ss += a[it][k] * a[it][k];
  float scale_b = 1.f;
  if (norm_branch) scale_b = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps_b);
  ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float v = a[it][k];
      if (norm_branch) v = v * scale_b * gb[it][k];
      xv[it][k] += v;
      ss += xv[it][k] * xv[it][k];
    }
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    if (i < hidden) Vec4<float>::store(xr + i, xv[it]);
  }
  if (!norm_out) return;
  const float scale_o = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps_o);
  T* out = h + (size_t)blockIdx.x * hidden;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    if (i >= hidden) continue;
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = xv[it][k] * scale_o * go[it][k];
    Vec4<T>::store(out + i, v);
  }
}

extern "C" int omnia_add_rmsnorm(float* x, const void* branch, const float* wb, float eps_b,
                                 int norm_branch, const float* wo, float eps_o, int norm_out,
                                 void* h, int rows, int hidden, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (hidden % 4 == 0 && hidden <= 8192) {
    const int threads = hidden <= 1024 ? 128 : hidden <= 4096 ? 256 : 512;
    const int iters = (hidden + threads * 4 - 1) / (threads * 4);
    OMNIA_DISPATCH_DTYPE(dtype, {
      if (iters <= 2)
        launch_pdl(add_rmsnorm_reg_kernel<T, 2>, rows, threads, 0, stream, 
            x, (const T*)branch, wb, eps_b, norm_branch, wo, eps_o, norm_out, (T*)h, hidden);
      else
        launch_pdl(add_rmsnorm_reg_kernel<T, 4>, rows, threads, 0, stream, 
            x, (const T*)branch, wb, eps_b, norm_branch, wo, eps_o, norm_out, (T*)h, hidden);
    });
    return OMNIA_LAUNCH_RESULT();
  }
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  OMNIA_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem);
    launch_pdl(add_rmsnorm_kernel<T>, rows, 256, smem, stream, x, (const T*)branch, wb, eps_b,
                                                       norm_branch, wo, eps_o, norm_out, (T*)h,
                                                       hidden);
  });
  return OMNIA_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------
// Per head of a projected row [.. q heads .. | .. k heads .. | .. v heads ..] (each
// group at its own column of `proj`): weightless RMS over the head (q and k; eps < 0
// skips it), half-split rotation of the first `rot` dims by angle pos * inv_freq[i]
// (inv_freq null: no rotation), then q goes to q_out and k, v go into cache pages
// [page][k|v][kv_head][offset][d] at slot_mapping[t] (slot < 0: nothing is stored).
// One warp per head, four heads per block; head_dim <= 256 and even.
template <typename T>
__global__ void qk_norm_rope_store_kernel(const T* __restrict__ proj, int row_stride, int q_col,
                                          int k_col, int v_col, int nq, int nkv, int d,
                                          float eps, const float* __restrict__ inv_freq, int rot,
                                          const int* __restrict__ positions,
                                          const long long* __restrict__ slot_mapping,
                                          T* __restrict__ q_out, T* __restrict__ pages,
                                          int page_size, long long num_slots, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hs = blockIdx.y * (blockDim.x >> 5) + warp;
  if (hs >= nq + 2 * nkv) return;
  const int kind = hs < nq ? 0 : (hs < nq + nkv ? 1 : 2);
  const int head = kind == 0 ? hs : (kind == 1 ? hs - nq : hs - nq - nkv);
  const T* src = proj + (size_t)t * row_stride + (kind == 0 ? q_col : kind == 1 ? k_col : v_col) +
                 (size_t)head * d;
  T* dst;
  if (kind == 0) {
    dst = q_out + ((size_t)t * nq + head) * d;
  } else {
    const long long slot = slot_mapping[t];
    if (slot < 0) return;
    if (slot >= num_slots) {
      if (lane == 0) atomicOr(err, OMNIA_ERR_SLOT);
      return;
    }
    const long long page = slot / page_size, off = slot % page_size;
    dst = pages + (((page * 2 + (kind == 2)) * nkv + head) * page_size + off) * d;
  }
  if (kind == 2) {
    for (int i = lane; i < d; i += 32) dst[i] = src[i];
    return;
  }
  // The head is staged in shared memory as float32: norm, then rotation, then one rounding.
  __shared__ float staged[4][256];
  float* v = staged[warp];
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float a = to_f32(src[i]);
    v[i] = a;
    ss += a * a;
  }
  float scale = 1.f;
  if (eps >= 0.f) scale = rsqrtf(warp_sum(ss) / (float)d + eps);
  __syncwarp();
  const int rhalf = inv_freq != nullptr ? rot / 2 : 0;
  const float pos = (float)positions[t];
  for (int i = lane; i < rhalf; i += 32) {
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    const float a = v[i] * scale, b = v[i + rhalf] * scale;
    dst[i] = from_f32<T>(a * c - b * s);
    dst[i + rhalf] = from_f32<T>(a * s + b * c);
  }
  for (int i = 2 * rhalf + lane; i < d; i += 32) dst[i] = from_f32<T>(v[i] * scale);
}

// The same step for head sizes that are multiples of 32 with full (or no) rotation: lane l owns
// VW = d / 32 contiguous dims, read and written as one vector; the rotation partner of a dim in
// the first half lives 16 lanes away.
template <typename T, int VW>
struct alignas(sizeof(T) * VW) HeadPack {
  T v[VW];
};

template <typename T, int VW>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_vec_kernel(const T* __restrict__ proj, int row_stride, int q_col, int k_col, int v_col, int nq,
                              int nkv, float eps, const float* __restrict__ inv_freq,
                              const int* __restrict__ positions, const long long* __restrict__ slot_mapping,
                              T* __restrict__ q_out, T* __restrict__ pages, int page_size, long long num_slots,
                              int* err) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int d = 32 * VW;
  __shared__ float cos_s[d / 2], sin_s[d / 2];
  const int t = blockIdx.x;  // one block per token: the token's angles are computed once for all heads
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (inv_freq != nullptr) {
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < d / 2; i += blockDim.x) sincosf(pos * inv_freq[i], &sin_s[i], &cos_s[i]);
  }
  __syncthreads();
  const long long slot = slot_mapping != nullptr ? slot_mapping[t] : -1;
  if (nkv > 0 && slot >= num_slots && threadIdx.x == 0) atomicOr(err, OMNIA_ERR_SLOT);
  for (int hs = warp; hs < nq + 2 * nkv; hs += blockDim.x >> 5) {
    const int kind = hs < nq ? 0 : (hs < nq + nkv ? 1 : 2);
    const int head = kind == 0 ? hs : (kind == 1 ? hs - nq : hs - nq - nkv);
    const T* src = proj + (size_t)t * row_stride + (kind == 0 ? q_col : kind == 1 ? k_col : v_col) + (size_t)head * d;
    T* dst;
    if (kind == 0) {
      dst = q_out + ((size_t)t * nq + head) * d;
    } else {
      if (slot < 0 || slot >= num_slots) continue;
      const long long page = slot / page_size, off = slot % page_size;
      dst = pages + (((page * 2 + (kind == 2)) * nkv + head) * page_size + off) * d;
    }
    HeadPack<T, VW> pack = *reinterpret_cast<const HeadPack<T, VW>*>(src + lane * VW);
    if (kind != 2) {
      float v[VW], ss = 0.f;
#pragma unroll
      for (int i = 0; i < VW; ++i) {
        v[i] = to_f32(pack.v[i]);
        ss += v[i] * v[i];
      }
      const float scale = eps >= 0.f ? rsqrtf(warp_sum(ss) / (float)d + eps) : 1.f;
#pragma unroll
      for (int i = 0; i < VW; ++i) {
        float mine = v[i] * scale;
        if (inv_freq != nullptr) {
          const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
          const float c = cos_s[(lane & 15) * VW + i], sn = sin_s[(lane & 15) * VW + i];
          mine = lane < 16 ? mine * c - other * sn : other * sn + mine * c;
        }
        pack.v[i] = from_f32<T>(mine);
      }
    }
    *reinterpret_cast<HeadPack<T, VW>*>(dst + lane * VW) = pack;
  }
}

extern "C" int omnia_qk_norm_rope_store(const void* proj, int row_stride, int q_col, int k_col,
                                        int v_col, int nq, int nkv, int d, float eps,
                                        const float* inv_freq, int rot, const int* positions,
                                        const long long* slot_mapping, void* q_out, void* pages,
                                        int page_size, long long num_slots, int tokens, int dtype,
                                        int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (d > 256 || (d & 1) || rot > d || (rot & 1)) return (int)cudaErrorInvalidValue;
  const int heads = nq + 2 * nkv;
  dim3 grid(tokens, (heads + 3) / 4);
  // Head sizes 64, 128, 256 with full or no rotation, and operands aligned for vector access.
  const bool vector_ok = (rot == d || inv_freq == nullptr) && (d == 64 || d == 128 || d == 256) &&
                         row_stride % 8 == 0 && q_col % 8 == 0 && k_col % 8 == 0 && v_col % 8 == 0 &&
                         ((uintptr_t)proj & 15) == 0 && ((uintptr_t)q_out & 15) == 0 && ((uintptr_t)pages & 15) == 0;
  if (vector_ok) {
    OMNIA_DISPATCH_DTYPE(dtype, {
      if (d == 64)
        launch_pdl(qk_norm_rope_store_vec_kernel<T, 2>, tokens, 256, 0, stream, (const T*)proj, row_stride, q_col, k_col,
                   v_col, nq, nkv, eps, inv_freq, positions, slot_mapping, (T*)q_out, (T*)pages, page_size, num_slots, err);
      else if (d == 128)
        launch_pdl(qk_norm_rope_store_vec_kernel<T, 4>, tokens, 256, 0, stream, (const T*)proj, row_stride, q_col, k_col,
                   v_col, nq, nkv, eps, inv_freq, positions, slot_mapping, (T*)q_out, (T*)pages, page_size, num_slots, err);
      else
        launch_pdl(qk_norm_rope_store_vec_kernel<T, 8>, tokens, 256, 0, stream, (const T*)proj, row_stride, q_col, k_col,
                   v_col, nq, nkv, eps, inv_freq, positions, slot_mapping, (T*)q_out, (T*)pages, page_size, num_slots, err);
    });
    return OMNIA_LAUNCH_RESULT();
  }
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(qk_norm_rope_store_kernel<T>, grid, 128, 0, stream, 
                                  (const T*)proj, row_stride, q_col, k_col, v_col, nq, nkv, d, eps,
                                  inv_freq, rot, positions, slot_mapping, (T*)q_out, (T*)pages,
                                  page_size, num_slots, err)));
  return OMNIA_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------
// angles[i][t] = (cos, sin)(positions[t] * inv_freq[i]): what a product's epilogue that rotates its
// own rows reads. It has a thread per row, so the tokens run along the table's rows: a warp's 32
// threads then read 32 neighbours. The same expression as in the kernel above, so a row rotates
// alike wherever it is rotated.
__global__ void rope_angles_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int half,
                                   int tokens, float2* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= (long long)tokens * half) return;
  const int t = (int)(index / half), i = (int)(index % half);
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
  out[(size_t)i * tokens + t] = make_float2(cs, sn);
}

extern "C" int omnia_rope_angles(const int* positions, const float* inv_freq, int half, int tokens, void* out,
                                 cudaStream_t stream) {
  const long long total = (long long)tokens * half;
  if (total == 0) return 0;
  launch_pdl(rope_angles_kernel, (int)((total + 255) / 256), 256, 0, stream, positions, inv_freq, half, tokens,
             (float2*)out);
  return OMNIA_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------
// act[t, i] = silu(gu[t, i]) * gu[t, inner + i], in float32, rounded once.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, long long total,
                              int inner) {
  pdl_wait();
  pdl_launch_dependents();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += stride) {
    const long long t = idx / inner;
    const int i = (int)(idx - t * inner);
    const float g = to_f32(gu[t * 2 * inner + i]);
    const float u = to_f32(gu[t * 2 * inner + inner + i]);
    act[idx] = from_f32<T>(g / (1.f + expf(-g)) * u);
  }
}

extern "C" int omnia_swiglu(const void* gu, void* act, int rows, int inner, int dtype,
                            cudaStream_t stream) {
  const long long total = (long long)rows * inner;
  if (total == 0) return 0;
  const long long most = 16LL * omnia_sm_count();
  const int blocks = (int)((total + 255) / 256 < most ? (total + 255) / 256 : most);
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(swiglu_kernel<T>, blocks, 256, 0, stream, 
                                  (const T*)gu, (T*)act, total, inner)));
  return OMNIA_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------
// logits = cap * tanh(z * multiplier / cap)  (cap <= 0: logits = z * multiplier), float32 out.
template <typename T>
__global__ void softcap_kernel(const T* __restrict__ z, float* __restrict__ out, long long total,
                               float multiplier, float cap) {
  pdl_wait();
  pdl_launch_dependents();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += stride) {
    const float v = to_f32(z[idx]) * multiplier;
    out[idx] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}

extern "C" int omnia_softcap(const void* z, float* out, long long total, float multiplier,
                             float cap, int dtype, cudaStream_t stream) {
  if (total == 0) return 0;
  const long long most = 16LL * omnia_sm_count();
  const int blocks = (int)((total + 255) / 256 < most ? (total + 255) / 256 : most);
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(softcap_kernel<T>, blocks, 256, 0, stream, (const T*)z, out,
                                                                            total, multiplier, cap)));
  return OMNIA_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------
// out[r] = src[rows[r]]  (rows of `width` elements)
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int* __restrict__ rows,
                                   T* __restrict__ out, int width) {
  pdl_wait();
  pdl_launch_dependents();
  const T* s = src + (size_t)rows[blockIdx.x] * width;
  T* o = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = s[i];
}

extern "C" int omnia_gather_rows(const void* src, const int* rows, void* out, int count, int width,
                                 int dtype, cudaStream_t stream) {
  if (count == 0) return 0;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(gather_rows_kernel<T>, count, 256, 0, stream, 
                                  (const T*)src, rows, (T*)out, width)));
  return OMNIA_LAUNCH_RESULT();
}
