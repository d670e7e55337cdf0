// Split of a step's fused q|k|v projection for attention without rotation: adds the
// projections' biases, separates q, k and v, and writes k and v into the paged cache.
//
// The projection row is [q_heads * d | kv_heads * d | kv_heads * dv]: values may have another
// width than queries and keys; dv = 0 is a projection without values (the values are the keys, or
// live inside them), and nothing is written through the value pointers. `bias` (float32, the row's width, or null) is added in float32
// before the result is rounded to the activation type. Cache layout: key pages
// [page][kv_head][page_size][d], value pages [page][kv_head][page_size][dv]; dest_rows[t] =
// page * page_size + row in page, or < 0 when the position is not kept (see rope_store.cu).
#include "common.cuh"

template <typename A>
__global__ void qkv_bias_store_kernel(const A* __restrict__ qkv, const float* __restrict__ bias,
                                      A* __restrict__ q_out, A* __restrict__ k_out,
                                      A* __restrict__ v_out, A* __restrict__ k_pages,
                                      A* __restrict__ v_pages, const int* __restrict__ dest_rows,
                                      int q_heads, int kv_heads, int d, int dv, int page_size) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int nq = q_heads * d, nk = kv_heads * d, nv = kv_heads * dv;
  const int width = nq + nk + nv;
  const A* src = qkv + static_cast<size_t>(t) * width;
  const int dest = k_pages != nullptr ? dest_rows[t] : -1;
  const long long page = dest >= 0 ? dest / page_size : -1;
  const int in_page = dest >= 0 ? dest % page_size : 0;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    float x = to_f32(src[c]);
    if (bias != nullptr) x += bias[c];
    const A val = from_f32<A>(x);
    if (c < nq) {
      q_out[static_cast<size_t>(t) * nq + c] = val;
    } else if (c < nq + nk) {
      const int e = c - nq, kh = e / d, j = e % d;
      if (k_out != nullptr) k_out[static_cast<size_t>(t) * nk + e] = val;
      if (page >= 0)
        k_pages[((static_cast<size_t>(page) * kv_heads + kh) * page_size + in_page) * d + j] = val;
    } else {
      const int e = c - nq - nk, kh = e / dv, j = e % dv;
      if (v_out != nullptr) v_out[static_cast<size_t>(t) * nv + e] = val;
      if (page >= 0)
        v_pages[((static_cast<size_t>(page) * kv_heads + kh) * page_size + in_page) * dv + j] = val;
    }
  }
}

LRM_API int lrm_qkv_bias_store(const void* qkv, int dtype, const float* bias, void* q_out, void* k_out,
                               void* v_out, void* k_pages, void* v_pages, const int* dest_rows,
                               int tokens, int q_heads, int kv_heads, int d, int dv, int page_size,
                               cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (q_heads <= 0 || kv_heads < 0 || d <= 0 || dv < 0 || page_size <= 0) return LRM_BAD_ARGUMENT;
  if (k_pages != nullptr && dest_rows == nullptr) return LRM_BAD_ARGUMENT;
  const int width = q_heads * d + kv_heads * (d + dv);
  const dim3 grid(tokens, (width + 1023) / 1024 > 0 ? (width + 1023) / 1024 : 1);
  if (dtype == LRM_F32)
    LRM_LAUNCH(qkv_bias_store_kernel<float>, grid, 256, 0, stream, static_cast<const float*>(qkv), bias,
               static_cast<float*>(q_out), static_cast<float*>(k_out), static_cast<float*>(v_out),
               static_cast<float*>(k_pages), static_cast<float*>(v_pages), dest_rows, q_heads, kv_heads, d,
               dv, page_size);
  else if (dtype == LRM_BF16)
    LRM_LAUNCH(qkv_bias_store_kernel<__nv_bfloat16>, grid, 256, 0, stream,
               static_cast<const __nv_bfloat16*>(qkv), bias, static_cast<__nv_bfloat16*>(q_out),
               static_cast<__nv_bfloat16*>(k_out), static_cast<__nv_bfloat16*>(v_out),
               static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages), dest_rows,
               q_heads, kv_heads, d, dv, page_size);
  else
    return LRM_BAD_ARGUMENT;
  return 0;
}
