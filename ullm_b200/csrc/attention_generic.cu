// Paged causal attention for any mix of requests in one flat batch: prompt
// portions of any length beside single decoded tokens.  This is the general
// kernel: any head size up to 512, any head counts, any page size, optional
// sliding window, float32 or bfloat16 storage.  It is the whole attention of
// the 32-bit path and the fallback of the bfloat16 path for sizes its
// tensor-core kernels do not take.
//
// One warp per (token, query head).  The query (scaled dot products in 32-bit)
// meets the keys 32 at a time, one key per lane; the running maximum, the
// running sum and the output accumulator are 32-bit (online softmax); exp is
// expf.  A token's keys are visited from the first visible position upward in
// groups of 32 counted from that position, so the result for a token does not
// depend on how the batch was cut, on the other requests in it, or on which
// pages hold the keys.
//
// Batch row r reads row req_slots[r] of the block table.  Request r owns query rows cu_q[r] .. cu_q[r+1]-1 and holds kv_len[r] tokens
// after this step; row j of it sits at position kv_len[r] - q_len[r] + j and
// sees positions max(0, pos - window + 1) .. pos (window 0 = all).
#include "common.cuh"

#define ATT_MAX_HEAD_DIM 512
#define ATT_WARPS 4
#define ATT_O_REGS (ATT_MAX_HEAD_DIM / 32)

template <typename T, int OREGS>
__global__ void paged_attention_generic_kernel(const T* __restrict__ q, long long q_row_stride, T* __restrict__ out,
                                               const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                               const int* __restrict__ block_table, int max_pages,
                                               const int* __restrict__ req_slots,
                                               const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                                               const int* __restrict__ token_req, int tokens, int num_q, int num_kv,
                                               int head_dim, int page_size, int window, float scale,
                                               long long num_pages, int* status) {
  __shared__ float qs[ATT_WARPS][ATT_MAX_HEAD_DIM];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * ATT_WARPS + warp;
  if (unit >= (long long)tokens * num_q) return;
  const int t = (int)(unit / num_q);
  const int h = (int)(unit - (long long)t * num_q);
  const int kh = h / (num_q / num_kv);
  T* o_ptr = out + ((long long)t * num_q + h) * head_dim;
  const int r = token_req[t];
  const int q_len = r >= 0 ? cu_q[r + 1] - cu_q[r] : 0;
  const int kvl = r >= 0 ? kv_len[r] : 0;
  const int pos = kvl - q_len + (r >= 0 ? t - cu_q[r] : 0);
  if (r < 0 || q_len <= 0 || kvl <= 0 || pos < 0) {  // padding row
    for (int e = lane; e < head_dim; e += 32) o_ptr[e] = from_f32<T>(0.f);
    return;
  }
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const T* q_ptr = q + (long long)t * q_row_stride + (long long)h * head_dim;
  float* qv = qs[warp];
  for (int e = lane; e < head_dim; e += 32) qv[e] = to_f32(q_ptr[e]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[OREGS];
#pragma unroll
  for (int i = 0; i < OREGS; ++i) acc[i] = 0.f;
  const int* bt = block_table + (long long)req_slots[r] * max_pages;
  const long long kv_row = (long long)num_kv * head_dim;

  for (int base = lo; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    long long slot = -1;
    float s = -INFINITY;
    if (valid) {
      const int page = bt[key / page_size];
      if (page < 0 || page >= num_pages) {
        ullm_report(status, ULLM_STATUS_PAGE, t, page);
      } else {
        slot = (long long)page * page_size + key % page_size;
        const T* kp = k_cache + slot * kv_row + (long long)kh * head_dim;
        float d = 0.f;
        for (int e = 0; e < head_dim; ++e) d += qv[e] * to_f32(kp[e]);
        s = d * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = (slot >= 0) ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);  // m = -inf on the first group: 0
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < OREGS; ++i) acc[i] *= alpha;
    const int n = min(32, pos - base + 1);
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long sj = __shfl_sync(0xffffffffu, slot, j);
      if (sj < 0) continue;
      const T* vp = v_cache + sj * kv_row + (long long)kh * head_dim;
#pragma unroll
      for (int i = 0; i < OREGS; ++i) {
        const int e = lane + 32 * i;
        if (e < head_dim) acc[i] += pj * to_f32(vp[e]);
      }
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < OREGS; ++i) {
    const int e = lane + 32 * i;
    if (e < head_dim) o_ptr[e] = from_f32<T>(acc[i] * inv);
  }
}

template <typename T>
static int launch_generic(const void* q, long long q_row_stride, void* out, const void* k_cache, const void* v_cache,
                          const int* block_table, int max_pages, const int* req_slots, const int* cu_q,
                          const int* kv_len, const int* token_req, int tokens, int num_q, int num_kv, int head_dim, int page_size,
                          int window, float scale, long long num_pages, int* status, cudaStream_t st) {
  const long long units = (long long)tokens * num_q;
  const long long blocks = (units + ATT_WARPS - 1) / ATT_WARPS;
  if (blocks > 0x7fffffffLL) return ULLM_ERR_BAD_SIZE;
#define LAUNCH(OREGS)                                                                                             \
  rc = ullm_launch_kernel(paged_attention_generic_kernel<T, OREGS>, dim3((int)blocks), dim3(ATT_WARPS * 32), 0, st, \
      (const T*)q, q_row_stride, (T*)out, (const T*)k_cache, (const T*)v_cache, block_table, max_pages, req_slots,  \
      cu_q, kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale, num_pages, status)
  int rc = ULLM_OK;
  if (head_dim <= 32) LAUNCH(1);
  else if (head_dim <= 64) LAUNCH(2);
  else if (head_dim <= 128) LAUNCH(4);
  else if (head_dim <= 256) LAUNCH(8);
  else LAUNCH(16);
#undef LAUNCH
  return rc;
}

extern "C" int ullm_paged_attention_generic(int dtype, const void* q, long long q_row_stride, void* out,
                                            const void* k_cache, const void* v_cache, const int* block_table,
                                            int max_pages, const int* req_slots, const int* cu_q, const int* kv_len,
                                            const int* token_req,
                                            int tokens, int num_q, int num_kv, int head_dim, int page_size, int window,
                                            float scale, long long num_pages, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_q <= 0 || num_kv <= 0 || head_dim <= 0 || page_size <= 0 || max_pages <= 0)
    return ULLM_ERR_BAD_SIZE;
  if (num_q % num_kv != 0 || head_dim > ATT_MAX_HEAD_DIM || window < 0) return ULLM_ERR_UNSUPPORTED;
  if (tokens == 0) return ULLM_OK;
  if (dtype == ULLM_DTYPE_F32)
    return launch_generic<float>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                 kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale, num_pages,
                                 status, st);
  if (dtype == ULLM_DTYPE_BF16)
    return launch_generic<__nv_bfloat16>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                         kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale,
                                         num_pages, status, st);
  if (dtype == ULLM_DTYPE_F16)
    return launch_generic<__half>(q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q,
                                  kv_len, token_req, tokens, num_q, num_kv, head_dim, page_size, window, scale, num_pages,
                                  status, st);
  return ULLM_ERR_BAD_DTYPE;
}
