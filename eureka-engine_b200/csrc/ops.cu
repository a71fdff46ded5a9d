// ops.cu -- format and activation-plane utility kernels.
#include "host.cuh"

// ---- activations -> fp16 planes ----------------------------------------------------------------
__global__ void k_xp_from_f32(const float *__restrict__ x, int K, int planes, XPlanes xp) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y, lane = threadIdx.x & 31;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) & ~31;
  if (c0 >= K) return;
  xp_store32(xp, t, planes, c0, x[(size_t)t * K + c0 + lane], lane);
}
__global__ void k_xp_from_bf16(const unsigned short *__restrict__ x, int K, XPlanes xp) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y, lane = threadIdx.x & 31;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) & ~31;
  if (c0 >= K) return;
  float v = __uint_as_float((uint32_t)x[(size_t)t * K + c0 + lane] << 16);
  xp_store32(xp, t, 1, c0, v, lane);
}
int ops_xp_from_f32(cudaStream_t s, const float *x, int T, int planes, XPlanes xp) {
  if (xp.K % 32) return llb_fail("xp: K %d", xp.K);
  if (T * planes > xp.NC) return llb_fail("xp: %d rows x %d planes do not fit %d columns", T, planes, xp.NC);
  CU_OK(llb_launch(k_xp_from_f32, dim3((xp.K + 255) / 256, T), dim3(256), (size_t)(0), s, x, xp.K, planes, xp));
  CU_OK(cudaGetLastError());
  return 0;
}
int ops_xp_from_bf16(cudaStream_t s, const void *x, int T, XPlanes xp) {
  if (xp.K % 32) return llb_fail("xp: K %d", xp.K);
  if (T > xp.NC) return llb_fail("xp: %d rows do not fit %d columns", T, xp.NC);
  CU_OK(llb_launch(k_xp_from_bf16, dim3((xp.K + 255) / 256, T), dim3(256), (size_t)(0), s, (const unsigned short *)x, xp.K, xp));
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- bit-exact row dequantisation (embedding rows; the dequant parity check) -------------------
__global__ void k_dequant_rows(int fmt, const uint8_t *__restrict__ W, int cols, const int *__restrict__ row_ids,
                               float *__restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int row = row_ids ? row_ids[r] : r;
  const uint8_t *src = W + (size_t)row * dev_row_bytes(fmt, cols);
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x)
    out[(size_t)r * cols + c] = deq_elem(fmt, src, cols, c);
}
int ops_dequant_rows(cudaStream_t s, int fmt, const uint8_t *W, int rows, int cols, const int *row_ids, int nrows,
                     float *out) {
  (void)rows;
  if (nrows < 1) return 0;
  int gx = (cols + 255) / 256;
  if (gx > 64) gx = 64;
  // gridDim.y is limited to 65535 rows per launch
  for (int r0 = 0; r0 < nrows; r0 += 65535) {
    int n = nrows - r0 < 65535 ? nrows - r0 : 65535;
    CU_OK(llb_launch(k_dequant_rows, dim3(gx, n), dim3(256), (size_t)(0), s, fmt, row_ids ? W : W + (size_t)r0 * dev_row_bytes(fmt, cols), cols,
                                              row_ids ? row_ids + r0 : nullptr, out + (size_t)r0 * cols));
    CU_OK(cudaGetLastError());
  }
  return 0;
}

// ---- Q6_K: 210-byte stored super-blocks -> 224-byte device super-blocks ------------------------
__global__ void k_repack_q6k(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, size_t nblocks) {
  pdl_trigger();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t n = nblocks * 224;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    size_t b = i / 224;
    int o = (int)(i - b * 224);
    dst[i] = o < 210 ? src[b * 210 + o] : 0;
  }
}
int ops_repack_q6k(cudaStream_t s, const uint8_t *src210, uint8_t *dst224, size_t nblocks) {
  if (!nblocks) return 0;
  size_t n = nblocks * 224;
  int grid = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  CU_OK(llb_launch(k_repack_q6k, dim3(grid), dim3(256), (size_t)(0), s, src210, dst224, nblocks));
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- fixed-order sum of K-slice partials --------------------------------------------------------
__global__ void k_sum_parts(const float *__restrict__ parts, int nsplit, long long stride, int n, float *__restrict__ out) {
  pdl_trigger();
  pdl_wait();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = parts[i];
  for (int k = 1; k < nsplit; k++) v += parts[(size_t)k * stride + i];
  out[i] = v;
}
int ops_sum_parts(cudaStream_t s, const float *parts, int nsplit, long long split_stride, int n, float *out) {
  CU_OK(llb_launch(k_sum_parts, dim3((n + 255) / 256), dim3(256), (size_t)(0), s, parts, nsplit, split_stride, n, out));
  CU_OK(cudaGetLastError());
  return 0;
}
