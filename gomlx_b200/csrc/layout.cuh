// Device-resident tile layout of GGML block-quantized weights.
//
// The bytes a caller uploads are the native GGML rows ([N, bytesPerRow] uint8,
// ml/ggml/dequant.go:31-35 in gomlx/gomlx).  On the device they are kept once, in a
// rearranged order that holds exactly the same bits: the matrix is cut into tiles of
// 16 rows x 256 values whose bytes are contiguous (2304 - 4352 bytes), tiles of one
// 16-row band follow each other along K.  A tile is what one TMA bulk copy moves into
// shared memory, and inside a tile the bytes are ordered so that the lanes of a warp read
// their pieces with conflict-free 128-bit shared loads:
//
//   per-row fields first, [row 0..15][16 bytes]   (block scales, super-block headers)
//   then "pieces" of 512 bytes, [lane 0..31][16 bytes]
//
// Lane l = 4*g + t of a warp feeds rows g and g+8 of the tile to the tensor cores and owns
// one quarter of the tile's 256 values.  Per format (r = 0 for row g, 1 for row g+8):
//
//   Q4_0  2304 B  [row][8 fp16 d]                  lane quarter t = blocks 2t, 2t+1
//                 piece 2*bp + r : the 16 nibble bytes of block 2t+bp
//   Q8_0  4352 B  [row][8 fp16 d]                  lane quarter t = blocks 2t, 2t+1
//                 piece 2*(2*bp + h) + r : int8 values 16h..16h+15 of block 2t+bp
//   Q4_K  2304 B  [row][d, dmin, scales[12]]       lane quarter t = sub-blocks 2t, 2t+1
//                 piece 2*i + r : bytes 32t+16i .. +16 of qs[128]
//   Q6_K  3360 B  [row][int8 scales[16]]           lane t = (n = t>>1, lh = t&1): values
//                 piece 0+r : ql[64n+16lh ..+16]         128n + 32c + 16lh + 0..15, c = 0..3
//                 piece 2+r : ql[64n+32+16lh ..+16]
//                 piece 4+r : qh[32n+16lh ..+16]
//                 then [row][fp16 d] (32 bytes)
//
// Rows beyond N and blocks beyond K are zero-filled (zero scale => zero weight).
#pragma once
#include <cstdint>

namespace b200q {

enum : int { kQ4_0 = 2, kQ8_0 = 8, kQ4_K = 12, kQ6_K = 14, kIQ4_NL = 20 };

constexpr int kTileRows = 16;
constexpr int kTileK = 256;

template <int TYPE>
struct Fmt;

template <>
struct Fmt<kQ4_0> {
    static constexpr int BPB = 18, VPB = 32, TK = kTileK, TILE = 2304;
    static constexpr int SUB = 32;       // values per aux sub-block (offset term granularity)
    static constexpr int AUX_PER_LANE = 2;
    static constexpr bool PERM4 = true;  // x staged as [x0,x2,x1,x3] per group of four
};
template <>
struct Fmt<kQ8_0> {
    static constexpr int BPB = 34, VPB = 32, TK = kTileK, TILE = 4352;
    static constexpr int SUB = 0;
    static constexpr int AUX_PER_LANE = 0;
    static constexpr bool PERM4 = false;
};
template <>
struct Fmt<kQ4_K> {
    static constexpr int BPB = 144, VPB = 256, TK = kTileK, TILE = 2304;
    static constexpr int SUB = 32;
    static constexpr int AUX_PER_LANE = 2;
    static constexpr bool PERM4 = true;
};
template <>
struct Fmt<kQ6_K> {
    static constexpr int BPB = 210, VPB = 256, TK = kTileK, TILE = 3360;
    static constexpr int SUB = 16;
    static constexpr int AUX_PER_LANE = 4;
    static constexpr bool PERM4 = false;
};

__host__ __device__ inline int fmt_bpb(int type) {
    return type == kQ4_0 ? 18 : type == kQ8_0 ? 34 : type == kQ4_K ? 144 : type == kQ6_K ? 210 : type == kIQ4_NL ? 18 : 0;
}
__host__ __device__ inline int fmt_vpb(int type) {
    return (type == kQ4_0 || type == kQ8_0 || type == kIQ4_NL) ? 32 : (type == kQ4_K || type == kQ6_K) ? 256 : 0;
}
__host__ __device__ inline int fmt_tile_bytes(int type) {
    return type == kQ4_0 ? Fmt<kQ4_0>::TILE : type == kQ8_0 ? Fmt<kQ8_0>::TILE : type == kQ4_K ? Fmt<kQ4_K>::TILE
                                                                                                : Fmt<kQ6_K>::TILE;
}

// Byte offset, inside a tile, of byte `o` (0..BPB-1) of block `b` (index inside the
// tile's K range) of tile row `r` (0..15).  This one function defines the layout:
// the upload kernel scatters with it, dequantize / embedding lookup gather with it.
template <int TYPE>
__host__ __device__ inline int tile_byte_offset(int r, int b, int o) {
    const int g = r & 7, rs = r >> 3;
    if constexpr (TYPE == kQ4_0) {
        const int t = b >> 1, bp = b & 1, lane = 4 * g + t;
        if (o < 2) return r * 16 + b * 2 + o;
        return 256 + (2 * bp + rs) * 512 + lane * 16 + (o - 2);
    } else if constexpr (TYPE == kQ8_0) {
        const int t = b >> 1, bp = b & 1, lane = 4 * g + t;
        if (o < 2) return r * 16 + b * 2 + o;
        const int q = o - 2, h = q >> 4;
        return 256 + (2 * (2 * bp + h) + rs) * 512 + lane * 16 + (q & 15);
    } else if constexpr (TYPE == kQ4_K) {
        if (o < 16) return r * 16 + o;
        const int q = o - 16, t = q >> 5, i = (q >> 4) & 1;
        return 256 + (2 * i + rs) * 512 + (4 * g + t) * 16 + (q & 15);
    } else {  // Q6_K
        if (o < 128) {  // ql
            const int n = o >> 6, w = o & 63, part = w >> 5, lh = (w >> 4) & 1;
            return 256 + (2 * part + rs) * 512 + (4 * g + 2 * n + lh) * 16 + (w & 15);
        }
        if (o < 192) {  // qh
            const int w = o - 128, n = w >> 5, lh = (w >> 4) & 1;
            return 256 + (4 + rs) * 512 + (4 * g + 2 * n + lh) * 16 + (w & 15);
        }
        if (o < 208) return r * 16 + (o - 192);  // scales
        return 3328 + r * 2 + (o - 208);         // d
    }
}

}  // namespace b200q
