// Token embedding: residual[t, :] = float32(table[ids[t], :]).
// A negative id is a placeholder for "the token this request sampled last": it is read
// from last_token[slot_of_token[t]], which the sampling kernels write on the device, so
// that a decode step can be launched before the host has seen the previous step's tokens.
// The residual stream is kept in 32-bit in both engine precisions, so the table
// row is widened here once.  An id outside [0, vocab) writes zeros and raises the
// error flag instead of reading out of bounds (the host checks ids first).
#include "common.cuh"
using namespace arle;

template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab,
                                 int* __restrict__ err, const int* __restrict__ last_token,
                                 const int* __restrict__ slot_of_token) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && last_token) id = last_token[slot_of_token[t]];
  float* o = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
    if (threadIdx.x == 0 && err) atomicExch(err, 1);
    return;
  }
  const T* row = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32(row[i]);
}

// Eight table elements per thread and step (16-byte loads of bfloat16 rows).
__global__ void embedding_bf16_vec_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                          float* __restrict__ out, int hidden, int vocab, int* __restrict__ err,
                                          const int* __restrict__ last_token, const int* __restrict__ slot_of_token) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && last_token) id = last_token[slot_of_token[t]];
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0 && err) atomicExch(err, 1);
  const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)(bad ? 0 : id) * hidden);
  float4* o = reinterpret_cast<float4*>(out + (size_t)t * hidden);
  for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) {
    uint4 u = make_uint4(0, 0, 0, 0);
    if (!bad) u = row[c];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    o[2 * c] = make_float4(__low2float(h[0]), __high2float(h[0]), __low2float(h[1]), __high2float(h[1]));
    o[2 * c + 1] = make_float4(__low2float(h[2]), __high2float(h[2]), __low2float(h[3]), __high2float(h[3]));
  }
}

ARLE_API int arle_embedding(const int* ids, const void* table, int table_dtype, float* out,
                            int num_tokens, int hidden, int vocab, int* err, const int* last_token,
                            const int* slot_of_token, cudaStream_t s) {
  if (last_token && !slot_of_token) return ARLE_E_BADARG;
  if (num_tokens <= 0) return 0;
  if (hidden <= 0 || vocab <= 0) return ARLE_E_BADARG;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == 1 && hidden % 8 == 0 && ((uintptr_t)table & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    int th = hidden / 8;
    th = th <= 32 ? 32 : (th <= 64 ? 64 : (th <= 128 ? 128 : (th <= 256 ? 256 : 512)));
    launch_kernel(embedding_bf16_vec_kernel, dim3(num_tokens), dim3(th), 0, s, 1, ids, (const __nv_bfloat16*)table, out, hidden, vocab, err, last_token, slot_of_token);
    return launch_status();
  }
  if (table_dtype == 0)
    launch_kernel(embedding_kernel<float>, dim3(num_tokens), dim3(threads), 0, s, 1, ids, (const float*)table, out, hidden, vocab, err, last_token, slot_of_token);
  else if (table_dtype == 1)
    launch_kernel(embedding_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, s, 1, ids, (const __nv_bfloat16*)table, out, hidden, vocab, err, last_token, slot_of_token);
  else
    return ARLE_E_BADARG;
  return launch_status();
}

// 1: kernels are launched so that the next kernel of the stream may start its set-up
// (barriers, weight prefetch) while the previous one finishes; 0 (default): plain launches.
ARLE_API void arle_set_programmatic_launch(int mode) { arle::pdl_enabled() = mode & 3; }
