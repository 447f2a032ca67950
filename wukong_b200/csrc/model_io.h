// Checkpoint containers: shared declarations of the host readers (model_io.cpp) and the device loaders
// (model_io_dev.cu).  Codes and dtype numbers are those of crates/wukong_runtime/src/fileio.rs:45-88.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace wkb_io {

enum : int64_t { DT_F32 = 0, DT_F64 = 1, DT_F16 = 2, DT_BF16 = 3, DT_I8 = 4, DT_I16 = 5, DT_I32 = 6, DT_I64 = 7,
                 DT_U8 = 8, DT_U16 = 9, DT_U32 = 10, DT_U64 = 11, DT_UNSUPPORTED = -1 };
enum : int64_t { IO_OPEN_FAILED = -1, IO_ERROR = -2, IO_DTYPE_MISMATCH = -3, IO_SHAPE_MISMATCH = -4, IO_NAME_NOT_FOUND = -5,
                 IO_BAD_HEADER = -6, IO_UNSUPPORTED_TYPE = -7 };

// One row of ggml's type table (crates/wukong_runtime/src/gguf.rs:244-289).
struct GgmlType {
  uint32_t id;
  const char* name;
  uint64_t block;     // elements per block (1 for a plain element type)
  uint64_t bytes;     // bytes per block
  int64_t dt;         // dtype code of a plain element type, DT_UNSUPPORTED for a block type
  bool dequant;       // a block type with a dequantizer
};
const GgmlType* ggml_type(uint32_t id);

// How a checked tensor moves into its destination (gguf.rs:652-663, fileio.rs:193-214).
enum class Move { Verbatim, Widen, Dequant, Raw };

// A named tensor located in a container and checked against a destination.
struct Located {
  Move move = Move::Verbatim;
  uint32_t ggml_id = 0;        // GGUF only
  int64_t src_dt = DT_UNSUPPORTED;   // the payload's dtype code (plain types)
  uint64_t data_off = 0, nbytes = 0;
  uint64_t count = 0;          // elements the read transfers
  std::vector<uint64_t> shape; // outermost first
};

int64_t dtype_size(int64_t dt);
// Open, parse, locate and plan: every check of the reference's order, before a byte of payload moves.
// dims == nullptr means a flat destination.  Returns 0 or a negative code.
int64_t gguf_locate_for(const char* path, const char* name, int64_t dest_dt, int64_t dest_len, const int64_t* dims, int64_t rank,
                        Located* out);
int64_t st_locate_for(const char* path, const char* name, int64_t dest_dt, int64_t dest_len, const int64_t* dims, int64_t rank,
                      Located* out);
// Dequantize one block of ggml type `id` (host; the arithmetic of ggml's dequantize_row_* in f32, each product
// and sum rounded once).
void dequant_block_host(uint32_t id, const uint8_t* blk, float* y);
float widen_half_host(uint16_t bits, int64_t src_dt);

}  // namespace wkb_io
