// A gated linear recurrence per channel, and the short causal convolution in front of it.
//
//   u_t   = conv(x)_t                      (short_conv: taps per channel, zeros before the start)
//   r_t   = sigmoid(gr_t),  i_t = sigmoid(gi_t)          (gate pre-activations come from products)
//   a_t   = exp(-rate_c * r_t)             (rate_c = factor * softplus(lam_c), made once on the host)
//   S_t   = a_t S_(t-1) + sqrt(1 - a_t^2) * (i_t * u_t)                 (S = 0 before the start)
//   out_t = S_t * gelu_tanh(y_t + by_c)
//
// Everything of the recurrence is float32: gates, decays, the state. The state S [slots, C] and
// the convolution's last n - 1 inputs [slots, n - 1, C] live in the cache's state storage and are
// carried from step to step, so a step of any size continues where the one before stopped.
// sqrt(1 - a^2) is formed as sqrt(-expm1(2 log a)), which keeps its digits when a is near 1.
// A sequence of padding (slot < 0) starts from zero and stores nothing.
//
// Two scan kernels. One thread per (sequence, channel) walks the step's tokens in order: decode
// steps and short portions. For long portions a CTA takes 32 channels of one sequence and cuts the
// portion into kChunks runs of tokens, one per warp-row: every run is scanned from zero while
// the product of its decays is kept, the runs' entry states follow from a short serial pass in
// shared memory, and every run is scanned again from its entry state, now writing outputs. The two
// ways differ only in rounding.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf(float z) { return 1.0f / (1.0f + expf(-z)); }

__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// One thread per (token, channel). Input x_t[c] = src[t, off + c] + in_bias[c]; inputs before the
// step come from `tails` (entry s is the input n - 1 - s tokens before the step's first), inputs
// before the sequence are zero. Taps [C, n]: the last column multiplies the current token.
template <typename S, typename O>
__global__ void short_conv_kernel(const S* __restrict__ src, long long stride, int off,
                                  const float* __restrict__ in_bias, const float* __restrict__ taps,
                                  const float* __restrict__ conv_bias, int n, const float* __restrict__ tails,
                                  const int* __restrict__ cu_seqlens, const int* __restrict__ seq_of_token,
                                  const int* __restrict__ slots, O* __restrict__ out, int C) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = seq_of_token[t], local = t - cu_seqlens[b], slot = slots[b];
  const float* tail = (slot >= 0 && n > 1) ? tails + static_cast<size_t>(slot) * (n - 1) * C : nullptr;
  const float bias = in_bias != nullptr ? in_bias[c] : 0.f;
  float acc = conv_bias != nullptr ? conv_bias[c] : 0.f;
  for (int back = n - 1; back >= 0; --back) {  // oldest input first
    const int at = local - back;
    float x;
    if (at >= 0)
      x = to_f32(src[static_cast<size_t>(t - back) * stride + off + c]) + bias;
    else
      x = tail != nullptr ? tail[static_cast<size_t>(n - 1 + at) * C + c] : 0.f;
    acc = fmaf(taps[static_cast<size_t>(c) * n + (n - 1 - back)], x, acc);
  }
  out[static_cast<size_t>(t) * C + c] = from_f32<O>(acc);
}

// After a step: every sequence's tail becomes the last n - 1 convolution inputs it has seen.
// One thread per (sequence, channel), entries ascending: entry s takes input m - (n - 1) + s of
// the step's m tokens, or, when that is before the step, the old entry s + m, which lies above
// every entry written so far.
template <typename S>
__global__ void short_conv_tail_kernel(const S* __restrict__ src, long long stride, int off,
                                       const float* __restrict__ in_bias, int C, int n, float* __restrict__ tails,
                                       const int* __restrict__ cu_seqlens, const int* __restrict__ slots) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = slots[b];
  if (c >= C || slot < 0) return;
  const int start = cu_seqlens[b], m = cu_seqlens[b + 1] - start;
  const float bias = in_bias != nullptr ? in_bias[c] : 0.f;
  float* tail = tails + static_cast<size_t>(slot) * (n - 1) * C;
  for (int s = 0; s < n - 1; ++s) {
    const int at = m - (n - 1) + s;
    tail[static_cast<size_t>(s) * C + c] =
        at >= 0 ? to_f32(src[static_cast<size_t>(start + at) * stride + off + c]) + bias
                : (s + m < n - 1 ? tail[static_cast<size_t>(s + m) * C + c] : 0.f);
  }
}

// What one token contributes: (decay a, input b) of S <- a S + b, and the read-out's factor.
template <typename U>
struct ScanInputs {
  const U* u;            // [T, C]
  const float* gates;    // [T, blocks, 2 * size]: a block's r pre-activations, then its i
  const float* y;        // [T, y_stride], the read-out branch before its bias and activation
  long long y_stride;
  int y_off;
  const float* y_bias;   // [C] or null
  const float* rate;     // [C]
  int C, size;

  __device__ __forceinline__ void step(int t, int c, float rate_c, float& a, float& b) const {
    const size_t g = static_cast<size_t>(t) * 2 * C + static_cast<size_t>(c / size) * 2 * size + c % size;
    const float r = sigmoidf(gates[g]), i = sigmoidf(gates[g + size]);
    const float log_a = -rate_c * r;
    a = expf(log_a);
    b = sqrtf(-expm1f(2.0f * log_a)) * (i * to_f32(u[static_cast<size_t>(t) * C + c]));
  }
  __device__ __forceinline__ float read_out(int t, int c, float state) const {
    const float z = y[static_cast<size_t>(t) * y_stride + y_off + c] + (y_bias != nullptr ? y_bias[c] : 0.f);
    return state * gelu_tanh(z);
  }
};

template <typename U, typename O>
__global__ void gated_scan_serial_kernel(ScanInputs<U> in, float* __restrict__ state, O* __restrict__ out,
                                         const int* __restrict__ cu_seqlens, const int* __restrict__ slots) {
  const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= in.C) return;
  const float rate_c = in.rate[c];
  pdl_trigger();
  pdl_wait();
  const int slot = slots[b];
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  float s = slot >= 0 ? state[static_cast<size_t>(slot) * in.C + c] : 0.f;
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    float a, x;
    in.step(t, c, rate_c, a, x);
    s = fmaf(a, s, x);
    out[static_cast<size_t>(t) * in.C + c] = from_f32<O>(in.read_out(t, c, s));
  }
  if (slot >= 0) state[static_cast<size_t>(slot) * in.C + c] = s;
}

constexpr int kChunks = 32;  // runs a long portion is cut into (warp-rows of a CTA)

template <typename U, typename O>
__global__ __launch_bounds__(32 * kChunks) void gated_scan_chunked_kernel(
    ScanInputs<U> in, float* __restrict__ state, O* __restrict__ out, const int* __restrict__ cu_seqlens,
    const int* __restrict__ slots) {
  __shared__ float decay[kChunks][32], carry[kChunks][32];
  const int b = blockIdx.y, c = blockIdx.x * 32 + threadIdx.x, run = threadIdx.y;
  const bool live = c < in.C;
  const float rate_c = live ? in.rate[c] : 0.f;
  pdl_wait();
  const int slot = slots[b];
  const int t0 = cu_seqlens[b], m = cu_seqlens[b + 1] - t0;
  const int per = (m + kChunks - 1) / kChunks;
  const int lo = t0 + min(m, run * per), hi = t0 + min(m, (run + 1) * per);
  float s = 0.f, prod = 1.f;
  if (live)
#pragma unroll 4
    for (int t = lo; t < hi; ++t) {
      float a, x;
      in.step(t, c, rate_c, a, x);
      s = fmaf(a, s, x);
      prod *= a;
    }
  decay[run][threadIdx.x] = prod;
  carry[run][threadIdx.x] = s;
  __syncthreads();
  if (run == 0 && live) {  // entry state of every run, in order
    float e = slot >= 0 ? state[static_cast<size_t>(slot) * in.C + c] : 0.f;
    for (int k = 0; k < kChunks; ++k) {
      const float next = fmaf(decay[k][threadIdx.x], e, carry[k][threadIdx.x]);
      carry[k][threadIdx.x] = e;
      e = next;
    }
    if (slot >= 0) state[static_cast<size_t>(slot) * in.C + c] = e;
  }
  __syncthreads();
  pdl_trigger();
  if (!live) return;
  s = carry[run][threadIdx.x];
#pragma unroll 4
  for (int t = lo; t < hi; ++t) {
    float a, x;
    in.step(t, c, rate_c, a, x);
    s = fmaf(a, s, x);
    out[static_cast<size_t>(t) * in.C + c] = from_f32<O>(in.read_out(t, c, s));
  }
}

template <typename U, typename O>
int launch_scan(ScanInputs<U> in, float* state, O* out, const int* cu_seqlens, const int* slots, int seqs,
                int longest, cudaStream_t stream) {
  if (longest >= 4 * kChunks) {
    LRM_LAUNCH((gated_scan_chunked_kernel<U, O>), dim3((in.C + 31) / 32, seqs), dim3(32, kChunks), 0, stream, in,
               state, out, cu_seqlens, slots);
  } else {
    const int threads = in.C >= 2048 ? 128 : 64;
    LRM_LAUNCH((gated_scan_serial_kernel<U, O>), dim3((in.C + threads - 1) / threads, seqs), threads, 0, stream, in,
               state, out, cu_seqlens, slots);
  }
  return 0;
}

}  // namespace

// out [T, C] (act dtype) = conv of the columns off .. off + C of src [T, stride] (float32 or act dtype)
// plus in_bias; then the tails take the step's last inputs (a second launch, when n > 1).
LRM_API int lrm_short_conv(const void* src, int src_dtype, long long stride, int off, const float* in_bias,
                           const float* taps, const float* conv_bias, int n, float* tails, const int* cu_seqlens,
                           const int* seq_of_token, const int* slots, void* out, int out_dtype, int tokens,
                           int seqs, int C, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (C <= 0 || n <= 0 || n > 64 || src == nullptr || taps == nullptr || out == nullptr) return LRM_BAD_ARGUMENT;
  if (n > 1 && tails == nullptr) return LRM_BAD_ARGUMENT;
  if (tokens > 65535 || seqs > 65535) return LRM_UNSUPPORTED;
  const dim3 grid((C + 127) / 128, tokens), tail_grid((C + 127) / 128, seqs);
#define LRM_CONV(ST, OT)                                                                                          \
  do {                                                                                                            \
    LRM_LAUNCH((short_conv_kernel<ST, OT>), grid, 128, 0, stream, static_cast<const ST*>(src), stride, off,       \
               in_bias, taps, conv_bias, n, static_cast<const float*>(tails), cu_seqlens, seq_of_token, slots,    \
               static_cast<OT*>(out), C);                                                                         \
    if (n > 1)                                                                                                    \
      LRM_LAUNCH((short_conv_tail_kernel<ST>), tail_grid, 128, 0, stream, static_cast<const ST*>(src), stride,    \
                 off, in_bias, C, n, tails, cu_seqlens, slots);                                                   \
    return 0;                                                                                                     \
  } while (0)
  if (src_dtype == LRM_F32 && out_dtype == LRM_F32) LRM_CONV(float, float);
  if (src_dtype == LRM_F32 && out_dtype == LRM_BF16) LRM_CONV(float, __nv_bfloat16);
  if (src_dtype == LRM_BF16 && out_dtype == LRM_BF16) LRM_CONV(__nv_bfloat16, __nv_bfloat16);
#undef LRM_CONV
  return LRM_BAD_ARGUMENT;
}

// The recurrence over a step's packed tokens; `longest` is the most tokens one sequence brings
// (launch geometry only). u and out have the activation type.
LRM_API int lrm_gated_linear_scan(const void* u, int dtype, const float* gates, const float* y, long long y_stride,
                                  int y_off, const float* y_bias, const float* rate, float* state, void* out,
                                  const int* cu_seqlens, const int* slots, int seqs, int longest, int C,
                                  int blocks, cudaStream_t stream) {
  if (seqs <= 0) return 0;
  if (C <= 0 || blocks <= 0 || C % blocks != 0 || u == nullptr || gates == nullptr || y == nullptr ||
      rate == nullptr || state == nullptr || out == nullptr)
    return LRM_BAD_ARGUMENT;
  if (seqs > 65535) return LRM_UNSUPPORTED;
  if (dtype == LRM_F32) {
    ScanInputs<float> in{static_cast<const float*>(u), gates, y, y_stride, y_off, y_bias, rate, C, C / blocks};
    return launch_scan(in, state, static_cast<float*>(out), cu_seqlens, slots, seqs, longest, stream);
  }
  if (dtype == LRM_BF16) {
    ScanInputs<__nv_bfloat16> in{static_cast<const __nv_bfloat16*>(u), gates, y, y_stride, y_off, y_bias, rate, C,
                                 C / blocks};
    return launch_scan(in, state, static_cast<__nv_bfloat16*>(out), cu_seqlens, slots, seqs, longest, stream);
  }
  return LRM_BAD_ARGUMENT;
}
