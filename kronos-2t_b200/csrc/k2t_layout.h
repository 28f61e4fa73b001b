// Device-side storage of quantized matrices ("8-row group records").
//
// The reference keeps weights in 16-row stripes tuned for NEON `tbl`/`sdot`
// (src/kernels/simd_lut.rs:3264-3400 for bit-planes, 4796-5023 for NF).  On the GPU the unit is an
// 8-row GROUP (one quarter-warp): for group g and 64-column chunk c there is one contiguous RECORD
// and a warp reads four consecutive records per step, so every 128-bit load of a quarter-warp
// covers one full 128-byte line.  Records of a group are contiguous over c, groups are contiguous
// over g: a CTA that owns a span of groups streams one linear byte range.
//
// Record contents (r = row in group 0..7, col = column in chunk 0..63):
//   nibble part (bit-plane low 4 bits, NF4/NF5 low 4 index bits): 256 B
//       byte  (col/32)*128 + r*16 + ((col%32)/8)*4 + ...   one 16-byte line per (half, row)
//       bit-plane: byte b = col%4 of word w = (col%32)/8, low nibble for (col%8)<4 else high nibble
//                  (so `word & 0x0F0F0F0F` is four consecutive columns, ready for dp4a)
//       NF:        nibble k = col%8 of word w (consecutive nibbles = prmt selectors)
//   +1 extra bit (5 planes, NF5): 64 B at 256: row r word (col/32) at 256 + r*8, bit 8*(col%4) + (col%32)/4
//   +2 extra bits (6 planes): 128 B at 256: row r word (col/16) at 256 + r*16, bits 8*(col%4) + 2*((col%16)/4)
//   NF3: 192 B: words W0..W3 at r*16 (+0..12), W4,W5 at 128 + r*8; columns 0..47 sit in the low
//        three bits of nibble (col%8) of word col/8; column 48+t (t<16) has index bit j in bit 3 of
//        nibble t%8 of word 3*(t/8) + j
//   E8Q2: 128 B: row r at r*16, byte 2*blk = template byte, 2*blk+1 = sign byte of columns 8*blk..8*blk+7
// Scales: one bf16 per (row, scale group), stored [group][scale group][row in group] after the
// records, so the eight lanes of a quarter-warp read 16 contiguous bytes per scale group.
// NF4 indices are re-encoded at upload: the 16 centroids are sorted ascending and the stored nibble is
// the rank of the centroid, so bit 3 of a nibble separates the eight largest from the eight smallest
// centroids (identity for the sorted codebooks the reference compiler emits).
// Rows beyond `rows` are padding: zero codes / index 0 and zero scales, never written to the output.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/kronos_cuda_ffi.h"

namespace k2t {

enum Format : uint32_t { FMT_BP4 = 0, FMT_BP5, FMT_BP6, FMT_NF4, FMT_NF3, FMT_NF5, FMT_E8Q2, FMT_COUNT };

struct MatrixGeom {
    Format fmt;
    uint32_t rows, cols, nc, sgc, nsg, ngroups, rec_bytes;
    int32_t max_odd;          // 2^B - 1 for bit-planes, 0 otherwise
    int8_t codebook32[32];    // expanded codebook (NF; NF4: sorted ascending), zero otherwise
    uint8_t nf4_rank[16];     // NF4: file index -> device nibble
    int32_t nf4_split_ok;     // NF4: 1 when the two-table decode applies (see k2t_gemv.cu)
    int32_t nf4_offset;       // NF4 two-table decode: centroid = table value + offset
    uint8_t nf4_hi[8];        // codebook32[8+l] - offset   (0..127)
    uint8_t nf4_lo[8];        // offset - codebook32[l]     (0..127)
    size_t rec_total;         // ngroups * nc * rec_bytes
    size_t scale_total;       // ngroups * 8 * nsg * 2
    size_t file_bytes;        // bytes of the matrix in the reference file format
};

// Validates `d` and fills `g`. Returns false and sets `err` on a malformed descriptor.
bool matrix_geometry(const KronosCudaMatrixDesc &d, MatrixGeom &g, std::string &err);

// Builds the device image (records followed by scales) in `out` (size rec_total + scale_total).
void repack_matrix(const KronosCudaMatrixDesc &d, const MatrixGeom &g, bool gate_up_interleave,
                   uint8_t *out, unsigned threads);

}  // namespace k2t
