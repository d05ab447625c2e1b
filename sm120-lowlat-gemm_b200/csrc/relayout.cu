// Load-time conversion of block-scale matrices between the row-major form the GEMM entry points take
// ([rows, K/16] bytes) and the tiled form in which checkpoints prepared for block-scaled tensor-core GEMMs store them:
// tiles of 128 rows x 4 scale columns, 512 contiguous bytes each, the byte of (row r, column c) of a tile at
// (r % 32) * 16 + (r / 32) * 4 + c, tiles ordered row tile major with rows and columns padded to whole tiles.
// Pure byte movement, HBM-bound: one CTA moves a 128-row x 128-column block through shared memory so that both the
// reads and the writes are contiguous.
#include "llg_internal.h"

namespace llg {

namespace {

constexpr int kTileRows = 128, kTileCols = 4, kTileBytes = 512;
constexpr int kTilesPerCta = 32;  // 128 scale columns per CTA

__device__ __forceinline__ int tiled_at(int r, int c) { return (r & 31) * 16 + (r >> 5) * 4 + c; }

__global__ void __launch_bounds__(256) sf_relayout_kernel(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                                                          int rows, int cols, int64_t ld, int to_tiled, int words) {
  __shared__ __align__(16) unsigned char buf[kTilesPerCta * kTileBytes];  // tiled order
  const int col_tiles = (cols + kTileCols - 1) / kTileCols;
  const int rt = blockIdx.y, ct0 = blockIdx.x * kTilesPerCta;
  const int nt = min(kTilesPerCta, col_tiles - ct0);
  const int64_t tiled_off = ((int64_t)rt * col_tiles + ct0) * kTileBytes;
  unsigned char* const lin_dst = dst;
  if (to_tiled) {
    // row-major -> shared memory (tiled order); bytes outside the matrix become zero
    for (int i = threadIdx.x; i < kTileRows * nt; i += blockDim.x) {
      const int r = i / nt, t = i - r * nt;  // consecutive threads: consecutive 4-byte groups of one row
      const int64_t row = (int64_t)rt * kTileRows + r;
      const int c0 = (ct0 + t) * kTileCols;
      unsigned char v[4] = {0, 0, 0, 0};
      if (row < rows) {
        if (words && c0 + 4 <= cols) {  // rows are 4-byte aligned: one load
          const uchar4 w = *reinterpret_cast<const uchar4*>(src + row * ld + c0);
          v[0] = w.x; v[1] = w.y; v[2] = w.z; v[3] = w.w;
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (c0 + c < cols) v[c] = src[row * ld + c0 + c];
        }
      }
      *reinterpret_cast<uchar4*>(buf + t * kTileBytes + tiled_at(r, 0)) = make_uchar4(v[0], v[1], v[2], v[3]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nt * kTileBytes / 16; i += blockDim.x)
      reinterpret_cast<uint4*>(dst + tiled_off)[i] = reinterpret_cast<const uint4*>(buf)[i];
  } else {
    for (int i = threadIdx.x; i < nt * kTileBytes / 16; i += blockDim.x)
      reinterpret_cast<uint4*>(buf)[i] = reinterpret_cast<const uint4*>(src + tiled_off)[i];
    __syncthreads();
    for (int i = threadIdx.x; i < kTileRows * nt; i += blockDim.x) {
      const int r = i / nt, t = i - r * nt;
      const int64_t row = (int64_t)rt * kTileRows + r;
      if (row >= rows) continue;
      const uchar4 v = *reinterpret_cast<const uchar4*>(buf + t * kTileBytes + tiled_at(r, 0));
      const unsigned char b[4] = {v.x, v.y, v.z, v.w};
      const int c0 = (ct0 + t) * kTileCols;
      if (words && c0 + 4 <= cols) {
        *reinterpret_cast<uchar4*>(lin_dst + row * ld + c0) = v;
        continue;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c0 + c < cols) lin_dst[row * ld + c0 + c] = b[c];
    }
  }
}

}  // namespace

cudaError_t sf_relayout_launch(const void* src, void* dst, int rows, int cols, int64_t ld, bool to_tiled, cudaStream_t s) {
  const int col_tiles = (cols + kTileCols - 1) / kTileCols, row_tiles = (rows + kTileRows - 1) / kTileRows;
  const dim3 grid((col_tiles + kTilesPerCta - 1) / kTilesPerCta, row_tiles, 1);
  const void* const lin = to_tiled ? src : dst;
  const int words = (ld % 4 == 0 && (reinterpret_cast<uintptr_t>(lin) & 3) == 0) ? 1 : 0;
  sf_relayout_kernel<<<grid, 256, 0, s>>>(static_cast<const unsigned char*>(src), static_cast<unsigned char*>(dst), rows, cols,
                                          ld, to_tiled ? 1 : 0, words);
  return cudaGetLastError();
}

}  // namespace llg
