// The three gather/copy operators of the reference's Copy extension
// (library/retroinfer/retroinfer_kernels/src/gather_copy.cu:25-96, :100-212, :216-283 with
// copy_kernel.cuh), for rows of 128 16-bit elements and pages ("units") of 8 rows.
// Every thread moves 16 bytes (the reference moves 8); index arrays and the second key/value
// source of the concat may live in pinned host memory and are then read through UVA.
#include "ri_common.cuh"

namespace {

constexpr int kUnit = 8;            // rows per page
constexpr int kPiecesPerRow = 16;   // 16-byte pieces per row

// rows indices[g, copy_start : copy_start+copy_num] of keys/values/metadata -> first copy_num rows of dst
__global__ void __launch_bounds__(256) gather_vectors_kernel(const uint4* __restrict__ ksrc, uint4* __restrict__ kdst,
                                                             const uint4* __restrict__ vsrc, uint4* __restrict__ vdst,
                                                             const uint16_t* __restrict__ msrc, uint16_t* __restrict__ mdst,
                                                             const int64_t* __restrict__ indices, int src_rows, int dst_rows,
                                                             int index_size, int copy_start, int copy_num) {
  const int g = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= copy_num * kPiecesPerRow) return;
  const int row = i >> 4, piece = i & 15;
  const int64_t src = indices[(int64_t)g * index_size + copy_start + row];
  if (src < 0 || src >= src_rows) return;                      // never read outside the source
  const int64_t s = ((int64_t)g * src_rows + src) * kPiecesPerRow + piece;
  const int64_t d = ((int64_t)g * dst_rows + row) * kPiecesPerRow + piece;
  kdst[d] = ksrc[s];
  vdst[d] = vsrc[s];
  if (piece == 0) mdst[(int64_t)g * dst_rows + row] = msrc[(int64_t)g * src_rows + src];
}

struct ConcatArgs {
  const uint4 *k1, *k2, *k3, *v1, *v2, *v3;
  uint4 *kd, *vd;
  const int32_t *idx2, *size2, *dst2, *chunks2, *idx3, *size3, *dst3, *chunks3;
  int32_t* valid;
  int64_t len1, len2, len3_units, buffer_rows;
  int index_length, copy_rows1;
  int ctas2;       // CTAs per group that move units of src2
};

// dst rows = src1[:copy_rows1] ++ listed units of src2 (vector-level start index) ++ listed units of
// src3 (unit-level index); only the first `size` rows of a unit are valid.
__global__ void __launch_bounds__(256) concat_kernel(ConcatArgs a) {
  const int g = blockIdx.y;
  const int n2 = a.chunks2[g], n3 = a.chunks3[g];
  const int64_t ib = (int64_t)g * a.index_length;
  const int total2 = n2 > 0 ? a.dst2[ib + n2 - 1] + a.size2[ib + n2 - 1] : 0;
  const int total3 = n3 > 0 ? a.dst3[ib + n3 - 1] + a.size3[ib + n3 - 1] : 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) a.valid[g] = a.copy_rows1 + total2 + total3;
  const int units1 = (a.copy_rows1 + kUnit - 1) / kUnit;
  const int sub = threadIdx.x >> 7, lane128 = threadIdx.x & 127;   // two units per pass, 128 pieces each
  const int row_in_unit = lane128 >> 4, piece = lane128 & 15;
  auto copy_unit = [&](const uint4* ks, const uint4* vs, int64_t src_row, int64_t dst_row, int valid_rows) {
    if (row_in_unit < valid_rows && src_row >= 0 && dst_row + row_in_unit < a.buffer_rows) {
      const int64_t s = (src_row + row_in_unit) * kPiecesPerRow + piece;
      const int64_t d = ((int64_t)g * a.buffer_rows + dst_row + row_in_unit) * kPiecesPerRow + piece;
      a.kd[d] = ks[s];
      a.vd[d] = vs[s];
    }
  };
  // units of src2: only the first `ctas2` CTAs of a group take part (pages in pinned host memory cross PCIe, where a
  // few CTAs keep the link full and a shallow request queue keeps other kernels' reads of pinned words fast)
  if ((int)blockIdx.x < a.ctas2) {
    const uint4* ks = a.k2 + (int64_t)g * a.len2 * kPiecesPerRow;
    const uint4* vs = a.v2 + (int64_t)g * a.len2 * kPiecesPerRow;
    for (int j = blockIdx.x * 2 + sub; j < n2; j += a.ctas2 * 2)
      copy_unit(ks, vs, a.idx2[ib + j], a.copy_rows1 + a.dst2[ib + j], a.size2[ib + j]);
  }
  // rows of src1 and units of src3: every CTA, starting with the CTAs that have no units of src2 to move
  const int n13 = units1 + n3;
  const int first = (blockIdx.x + gridDim.x - a.ctas2 % gridDim.x) % gridDim.x;
  for (int u = first * 2 + sub; u < n13; u += gridDim.x * 2) {
    if (u < units1) {
      copy_unit(a.k1 + (int64_t)g * a.len1 * kPiecesPerRow, a.v1 + (int64_t)g * a.len1 * kPiecesPerRow, (int64_t)u * kUnit,
                (int64_t)u * kUnit, min(kUnit, a.copy_rows1 - u * kUnit));
    } else {
      const int j = u - units1;
      copy_unit(a.k3 + (int64_t)g * a.len3_units * kUnit * kPiecesPerRow, a.v3 + (int64_t)g * a.len3_units * kUnit * kPiecesPerRow,
                (int64_t)a.idx3[ib + j] * kUnit, a.copy_rows1 + total2 + a.dst3[ib + j], a.size3[ib + j]);
    }
  }
}

// for each listed unit: `size` rows starting at copy_start + src_idx of the source -> first rows of
// destination unit dst_idx
__global__ void __launch_bounds__(256) scatter_kernel(const uint4* __restrict__ ks, uint4* __restrict__ kd,
                                                      const uint4* __restrict__ vs, uint4* __restrict__ vd,
                                                      const int32_t* __restrict__ src_idx, const int32_t* __restrict__ sizes,
                                                      const int32_t* __restrict__ dst_idx, const int32_t* __restrict__ chunks,
                                                      int64_t src_rows, int64_t dst_units, int index_length, int copy_start) {
  const int g = blockIdx.y;
  const int n = chunks[g];
  const int64_t ib = (int64_t)g * index_length;
  const int sub = threadIdx.x >> 7, lane128 = threadIdx.x & 127;
  const int row_in_unit = lane128 >> 4, piece = lane128 & 15;
  for (int u = blockIdx.x * 2 + sub; u < n; u += gridDim.x * 2) {
    const int64_t src_row = (int64_t)copy_start + src_idx[ib + u];
    const int64_t du = dst_idx[ib + u];
    if (row_in_unit < sizes[ib + u] && du >= 0 && du < dst_units && src_row + row_in_unit < src_rows) {
      const int64_t s = ((int64_t)g * src_rows + src_row + row_in_unit) * kPiecesPerRow + piece;
      const int64_t d = (((int64_t)g * dst_units + du) * kUnit + row_in_unit) * kPiecesPerRow + piece;
      kd[d] = ks[s];
      vd[d] = vs[s];
    }
  }
}

}  // namespace

extern "C" int ri_gather_copy_vectors(const void* key_data, void* key_buffer, const void* value_data, void* value_buffer,
                                      const void* src_metadata, void* dst_metadata, const int64_t* data_offsets,
                                      int32_t groups, int32_t data_length, int32_t buffer_length, int32_t index_size,
                                      int32_t copy_start, int32_t copy_num, void* stream) {
  RI_REQUIRE(key_data && key_buffer && value_data && value_buffer && src_metadata && dst_metadata && data_offsets,
             "ri_gather_copy_vectors: null pointer");
  RI_REQUIRE(groups > 0 && groups <= 65535 && data_length > 0 && buffer_length > 0, "ri_gather_copy_vectors: bad sizes");
  RI_REQUIRE(copy_num >= 0 && copy_num <= buffer_length && copy_start >= 0 && copy_start + copy_num <= index_size,
             "ri_gather_copy_vectors: copy range [%d, %d) outside the index (%d) or the buffer (%d)", copy_start,
             copy_start + copy_num, index_size, buffer_length);
  if (copy_num == 0) return RI_OK;
  dim3 grid((copy_num * kPiecesPerRow + 255) / 256, groups);
  gather_vectors_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(key_data), static_cast<uint4*>(key_buffer), static_cast<const uint4*>(value_data),
      static_cast<uint4*>(value_buffer), static_cast<const uint16_t*>(src_metadata), static_cast<uint16_t*>(dst_metadata),
      data_offsets, data_length, buffer_length, index_size, copy_start, copy_num);
  RI_LAUNCH_OK("gather_vectors_kernel");
  return RI_OK;
}

extern "C" int ri_gather_copy_and_concat(const void* key_data1, const void* key_data2, const void* key_data3,
                                         void* key_buffer, const void* value_data1, const void* value_data2,
                                         const void* value_data3, void* value_buffer, const int32_t* data_offsets2,
                                         const int32_t* data_copy_sizes2, const int32_t* buffer_offsets2,
                                         const int32_t* copy_chunks2, const int32_t* data_offsets3,
                                         const int32_t* data_copy_sizes3, const int32_t* buffer_offsets3,
                                         const int32_t* copy_chunks3, int32_t* valid_lengths, int32_t groups,
                                         int32_t data_length1, int64_t data_length2, int32_t data_length3,
                                         int32_t buffer_length, int32_t offset_length, int32_t copy_vectors1,
                                         void* stream) {
  RI_REQUIRE(key_data1 && key_data2 && key_data3 && key_buffer && value_data1 && value_data2 && value_data3 &&
                 value_buffer && data_offsets2 && data_copy_sizes2 && buffer_offsets2 && copy_chunks2 && data_offsets3 &&
                 data_copy_sizes3 && buffer_offsets3 && copy_chunks3 && valid_lengths,
             "ri_gather_copy_and_concat: null pointer");
  RI_REQUIRE(groups > 0 && groups <= 65535 && offset_length > 0 && buffer_length > 0, "ri_gather_copy_and_concat: bad sizes");
  RI_REQUIRE(copy_vectors1 >= 0 && copy_vectors1 <= data_length1 && copy_vectors1 <= buffer_length,
             "ri_gather_copy_and_concat: copy_vectors1=%d exceeds source (%d) or buffer (%d)", copy_vectors1, data_length1,
             buffer_length);
  ConcatArgs a;
  a.k1 = static_cast<const uint4*>(key_data1); a.k2 = static_cast<const uint4*>(key_data2);
  a.k3 = static_cast<const uint4*>(key_data3); a.kd = static_cast<uint4*>(key_buffer);
  a.v1 = static_cast<const uint4*>(value_data1); a.v2 = static_cast<const uint4*>(value_data2);
  a.v3 = static_cast<const uint4*>(value_data3); a.vd = static_cast<uint4*>(value_buffer);
  a.idx2 = data_offsets2; a.size2 = data_copy_sizes2; a.dst2 = buffer_offsets2; a.chunks2 = copy_chunks2;
  a.idx3 = data_offsets3; a.size3 = data_copy_sizes3; a.dst3 = buffer_offsets3; a.chunks3 = copy_chunks3;
  a.valid = valid_lengths;
  a.len1 = data_length1; a.len2 = data_length2; a.len3_units = data_length3; a.buffer_rows = buffer_length;
  a.index_length = offset_length; a.copy_rows1 = copy_vectors1;
  cudaPointerAttributes attr;
  const bool host_pages = cudaPointerGetAttributes(&attr, key_data2) == cudaSuccess && attr.type == cudaMemoryTypeHost;
  (void)cudaGetLastError();
  a.ctas2 = host_pages ? 2 : 16;
  concat_kernel<<<dim3(16, groups), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  RI_LAUNCH_OK("concat_kernel");
  return RI_OK;
}

// One strided host-to-device copy per tensor: the first `rows` rows of every group's slot of the staging area
// (what ri_wb_stage_misses filled) go to the same place of the device-side staging buffers.
extern "C" int ri_stage_upload(void* d_stage_keys, void* d_stage_values, const void* h_stage_keys, const void* h_stage_values,
                               int32_t groups, int64_t stage_rows_per_group, int32_t rows, int32_t row_bytes, void* stream) {
  RI_REQUIRE(d_stage_keys && d_stage_values && h_stage_keys && h_stage_values, "ri_stage_upload: null pointer");
  RI_REQUIRE(groups > 0 && stage_rows_per_group > 0 && row_bytes > 0 && rows >= 0 && rows <= stage_rows_per_group,
             "ri_stage_upload: bad sizes");
  if (rows == 0) return RI_OK;
  const size_t pitch = (size_t)stage_rows_per_group * row_bytes, width = (size_t)rows * row_bytes;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RI_CUDA_OK(cudaMemcpy2DAsync(d_stage_keys, pitch, h_stage_keys, pitch, width, groups, cudaMemcpyHostToDevice, s));
  RI_CUDA_OK(cudaMemcpy2DAsync(d_stage_values, pitch, h_stage_values, pitch, width, groups, cudaMemcpyHostToDevice, s));
  return RI_OK;
}

extern "C" int ri_gather_copy_and_scatter(const void* key_data, void* key_buffer, const void* value_data,
                                          void* value_buffer, const int32_t* s_offsets, const int32_t* copy_sizes,
                                          const int32_t* d_offsets, const int32_t* copy_chunks, int32_t groups,
                                          int32_t data_length, int32_t buffer_length, int32_t offset_length,
                                          int32_t s_copy_start, void* stream) {
  RI_REQUIRE(key_data && key_buffer && value_data && value_buffer && s_offsets && copy_sizes && d_offsets && copy_chunks,
             "ri_gather_copy_and_scatter: null pointer");
  RI_REQUIRE(groups > 0 && groups <= 65535 && data_length > 0 && buffer_length > 0 && offset_length > 0 && s_copy_start >= 0,
             "ri_gather_copy_and_scatter: bad sizes");
  scatter_kernel<<<dim3(8, groups), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(key_data), static_cast<uint4*>(key_buffer), static_cast<const uint4*>(value_data),
      static_cast<uint4*>(value_buffer), s_offsets, copy_sizes, d_offsets, copy_chunks, data_length, buffer_length,
      offset_length, s_copy_start);
  RI_LAUNCH_OK("scatter_kernel");
  return RI_OK;
}
