// Device layout of a quantised weight matrix ("fragment tiles").
//
// tang-infer keeps a weight as an array of {scale, 32 values} blocks (crates/tang-infer/src/
// quantize.rs:15-31).  For the GPU the same numbers are regrouped, once, at upload, so that
//   * the bytes one CTA needs for one pipeline stage are CONTIGUOUS in HBM (one bulk copy), and
//   * every lane of a warp finds the operands of its tensor-core fragment as 16-byte vectors.
// No value changes: nibbles stay q+8, int8 stay int8, scales keep their bits.
//
// A tile covers 16 output rows x 128 k (four 32-blocks per row).  Tiles are stored [row block]
// [k chunk].  Inside a tile, for lane L = 4*g + t (g = row in 0..7, t = k quarter in 0..3) and
// half h (rows g and g+8):
//   Q4 : 16 bytes at  h*512 + 16*L : four 32-bit words, word j = block j's eight nibbles for
//        k = 32*j + 8*t + {0,2,4,6,1,3,5,7} (nibble 0 first).  That order makes the in-register
//        dequantiser emit (k0,k1) (k2,k3) (k4,k5) (k6,k7) pairs, which is how the activation
//        fragment of mma.m16n8k16 is laid out — so activations need no shuffling.
//   I8 : two planes p (blocks 2p, 2p+1): 16 bytes at h*1024 + p*512 + 16*L = for each of the two
//        blocks, bytes k = 8*t + {0,2,4,6} then {1,3,5,7}.
//   scales (after the weights): f16: h*64 + g*8 + 2*j ; f32: h*128 + g*16 + 4*j.
// Rows and k beyond the matrix are padded with q = 0 and scale = 0.
#pragma once

#include <stddef.h>
#include <stdint.h>

namespace tq {

enum QKind : int { Q4_F32 = 0, Q4_F16 = 1, Q8_F32 = 2, I8_ROW = 3 };

constexpr int kTileRows = 16;
constexpr int kTileK = 128;

__host__ __device__ inline bool qk_is8(int kind) { return kind == Q8_F32 || kind == I8_ROW; }
__host__ __device__ inline int qk_weight_bytes(int kind) { return qk_is8(kind) ? 2048 : 1024; }
__host__ __device__ inline int qk_scale_bytes(int kind) {
  return kind == Q4_F16 ? 128 : kind == I8_ROW ? 0 : 256;
}
__host__ __device__ inline int qk_tile_bytes(int kind) { return qk_weight_bytes(kind) + qk_scale_bytes(kind); }

// Byte offset of the scale of (local row r, block j) inside a tile.
__host__ __device__ inline int qk_scale_offset(int kind, int r, int j) {
  const int h = r >> 3, g = r & 7;
  return kind == Q4_F16 ? qk_weight_bytes(kind) + h * 64 + g * 8 + 2 * j : qk_weight_bytes(kind) + h * 128 + g * 16 + 4 * j;
}

}  // namespace tq
