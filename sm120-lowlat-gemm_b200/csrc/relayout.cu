// Load-time conversion of block-scale matrices between the row-major form the GEMM entry points take
// ([rows, K/16] bytes) and the tiled form in which checkpoints prepared for block-scaled tensor-core GEMMs store them:
// tiles of 128 rows x 4 scale columns, 512 contiguous bytes each, the byte of (row r, column c) of a tile at
// (r % 32) * 16 + (r / 32) * 4 + c, tiles ordered row tile major with rows and columns padded to whole tiles.
// Pure byte movement, run once per weight at load time: one CTA moves a 128-row x 128-column block through shared memory so that both the
// reads and the writes are contiguous (the tiled buffer needs 16-byte alignment, hence whole words on that side).
#include "llg_internal.h"

namespace llg {

namespace {

constexpr int kTileRows = 128, kTileCols = 4, kTileBytes = 512;
constexpr int kTilesPerCta = 32;  // 128 scale columns per CTA

constexpr int kTileWords = kTileBytes / 4, kTilePitch = kTileWords + 1;  // +1 word: a warp's 32 tiles fall on 32 banks

__global__ void __launch_bounds__(256) sf_relayout_kernel(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                                                          int rows, int cols, int64_t ld, int to_tiled, int words) {
  // tiles in tiled word order, one padding word between tiles: the row-major side walks a row across the tiles
  // (word (r % 32) * 4 + r / 32 of every tile), the tiled side walks the words of a tile
  __shared__ uint32_t buf[kTilesPerCta * kTilePitch];
  const int col_tiles = (cols + kTileCols - 1) / kTileCols;
  const int rt = blockIdx.y, ct0 = blockIdx.x * kTilesPerCta;
  const int nt = min(kTilesPerCta, col_tiles - ct0);
  const int64_t tiled_word0 = ((int64_t)rt * col_tiles + ct0) * kTileWords;
  if (to_tiled) {
    // row-major -> shared memory; bytes outside the matrix become zero
    for (int i = threadIdx.x; i < kTileRows * nt; i += blockDim.x) {
      const int r = i / nt, t = i - r * nt;  // consecutive threads: consecutive 4-byte groups of one row
      const int64_t row = (int64_t)rt * kTileRows + r;
      const int c0 = (ct0 + t) * kTileCols;
      uint32_t v = 0u;
      if (row < rows) {
        if (words && c0 + 4 <= cols) {  // rows are 4-byte aligned: one load
          v = *reinterpret_cast<const uint32_t*>(src + row * ld + c0);
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (c0 + c < cols) v |= (uint32_t)src[row * ld + c0 + c] << (8 * c);
        }
      }
      buf[t * kTilePitch + (r & 31) * 4 + (r >> 5)] = v;
    }
    __syncthreads();
    uint32_t* const out = reinterpret_cast<uint32_t*>(dst) + tiled_word0;
    for (int i = threadIdx.x; i < nt * kTileWords; i += blockDim.x) out[i] = buf[(i / kTileWords) * kTilePitch + i % kTileWords];
  } else {
    const uint32_t* const in = reinterpret_cast<const uint32_t*>(src) + tiled_word0;
    for (int i = threadIdx.x; i < nt * kTileWords; i += blockDim.x) buf[(i / kTileWords) * kTilePitch + i % kTileWords] = in[i];
    __syncthreads();
    for (int i = threadIdx.x; i < kTileRows * nt; i += blockDim.x) {
      const int r = i / nt, t = i - r * nt;
      const int64_t row = (int64_t)rt * kTileRows + r;
      if (row >= rows) continue;
      const uint32_t v = buf[t * kTilePitch + (r & 31) * 4 + (r >> 5)];
      const int c0 = (ct0 + t) * kTileCols;
      if (words && c0 + 4 <= cols) {
        *reinterpret_cast<uint32_t*>(dst + row * ld + c0) = v;
        continue;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c0 + c < cols) dst[row * ld + c0 + c] = (unsigned char)(v >> (8 * c));
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
