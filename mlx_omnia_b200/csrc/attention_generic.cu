// Paged causal attention for any batch shape, head size (<= 256), page size and element
// type: the kernel of the 32-bit path, and of sizes the tiled kernels refuse.
//
// One warp per (token, query head). Keys are visited in chunks of 32 starting at the
// lowest visible position; in a chunk every lane scores one key (a full dot product in
// float32), the chunk's softmax statistics are merged online, and for the values every
// lane owns the output dims lane, lane+32, ... The order of all additions depends only on
// the token's own position and window, never on how the batch was cut.
#include "common.cuh"

template <typename T>
__global__ void paged_attention_generic_kernel(
    const T* __restrict__ q,                // [tokens, nq, d]
    const T* __restrict__ pages,            // [num_pages, 2, nkv, page_size, d]
    const int* __restrict__ block_table,    // [num_seqs, max_pages]
    const int* __restrict__ cu_seqlens,     // [num_seqs + 1]
    const int* __restrict__ positions,      // [tokens]
    const T* __restrict__ gate, int gate_stride,  // gate[t * gate_stride + h * d + i], or null
    T* __restrict__ out,                    // [tokens, nq * d]
    int num_seqs, int max_pages, int num_pages, int nq, int nkv, int d, int page_size,
    int window, float scale, int* err) {
  __shared__ float qs[4][256];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * 4 + warp;
  if (head >= nq) return;
  // The request this token belongs to: the last s with cu_seqlens[s] <= t.
  int lo_s = 0, hi_s = num_seqs - 1;
  while (lo_s < hi_s) {
    const int mid = (lo_s + hi_s + 1) >> 1;
    if (cu_seqlens[mid] <= t) lo_s = mid; else hi_s = mid - 1;
  }
  const int seq = lo_s;
  const int pos = positions[t];
  const int kvh = head / (nq / nkv);
  const int first = window > 0 ? max(0, pos - window + 1) : 0;

  const T* qrow = q + ((size_t)t * nq + head) * d;
  for (int i = lane; i < d; i += 32) qs[warp][i] = to_f32(qrow[i]) * scale;
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  const int* table = block_table + (size_t)seq * max_pages;

  for (int base = first; base <= pos; base += 32) {
    const int j = base + lane;
    float s = -INFINITY;
    long long vrow = -1;
    if (j <= pos) {
      const int page = table[j / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, OMNIA_ERR_PAGE);
      } else {
        const long long krow = (((long long)page * 2) * nkv + kvh) * page_size + j % page_size;
        vrow = krow + (long long)nkv * page_size;
        const T* kp = pages + krow * d;
        float dot = 0.f;
        for (int i = 0; i < d; ++i) dot += qs[warp][i] * to_f32(kp[i]);
        s = dot;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float alpha = expf(m - m_new);
    const float p = s == -INFINITY ? 0.f : expf(s - m_new);
    l = l * alpha + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] *= alpha;
    const int count = min(32, pos - base + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long vr = __shfl_sync(0xffffffffu, vrow, jj);
      if (vr < 0) continue;
      const T* vp = pages + vr * d;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int i = lane + 32 * k;
        if (i < d) acc[k] += pj * to_f32(vp[i]);
      }
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* orow = out + ((size_t)t * nq + head) * d;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int i = lane + 32 * k;
    if (i >= d) continue;
    float v = acc[k] * inv;
    if (gate != nullptr) {
      const float g = to_f32(gate[(size_t)t * gate_stride + (size_t)head * d + i]);
      v *= 1.f / (1.f + expf(-g));
    }
    orow[i] = from_f32<T>(v);
  }
}

extern "C" int omnia_paged_attention_generic(
    const void* q, const void* pages, const int* block_table, const int* cu_seqlens,
    const int* positions, const void* gate, int gate_stride, void* out, int tokens, int num_seqs,
    int max_pages, int num_pages, int nq, int nkv, int d, int page_size, int window, float scale,
    int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (d > 256 || nkv <= 0 || nq % nkv != 0) return (int)cudaErrorInvalidValue;
  dim3 grid(tokens, (nq + 3) / 4);
  OMNIA_DISPATCH_DTYPE(dtype, (paged_attention_generic_kernel<T><<<grid, 128, 0, stream>>>(
                                  (const T*)q, (const T*)pages, block_table, cu_seqlens, positions,
                                  (const T*)gate, gate_stride, (T*)out, num_seqs, max_pages,
                                  num_pages, nq, nkv, d, page_size, window, scale, err)));
  return OMNIA_LAUNCH_RESULT();
}
