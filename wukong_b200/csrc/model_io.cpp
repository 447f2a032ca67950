// Checkpoint readers on the host: GGUF (versions 2 and 3) and safetensors.
//
// These are the reference's `gguf_read_<T>` / `gguf_find|rank|dim|type` / `gguf_meta_*` / `st_read_<T>` runtime
// entries (crates/wukong_runtime/src/gguf.rs:809-1110, crates/wukong_runtime/src/safetensors.rs:379-407) with the
// same names, arguments, check order and result codes (crates/wukong_runtime/src/fileio.rs:45-88, 193-243).
// The device loaders in model_io_dev.cu reuse the parse / locate / plan half and move the payload to the GPU
// as raw bytes, where it is dequantized.
//
// The container formats are public (ggml's GGUF specification and type table; the safetensors header layout);
// the block formats are ggml's `block_q*` structures, dequantized with ggml's reference arithmetic in f32.
#include "model_io.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <set>
#include <sys/stat.h>

namespace wkb_io {

// ---------------------------------------------------------------------------------------------------------
// scalars
// ---------------------------------------------------------------------------------------------------------
static float f32_from_bits(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  if (exp == 0) {
    if (man == 0) return f32_from_bits(sign);
    int e = -1;                       // subnormal half: normalise
    do { man <<= 1; ++e; } while (!(man & 0x400u));
    return f32_from_bits(sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13));
  }
  if (exp == 31) return f32_from_bits(sign | 0x7F800000u | (man << 13));
  return f32_from_bits(sign | ((exp + 112u) << 23) | (man << 13));
}
float widen_half_host(uint16_t bits, int64_t src_dt) {
  if (src_dt == DT_BF16) return f32_from_bits((uint32_t)bits << 16);
  if (src_dt == DT_F16) return f16_to_f32(bits);
  return NAN;
}
int64_t dtype_size(int64_t dt) {
  switch (dt) {
    case DT_I8: case DT_U8: return 1;
    case DT_F16: case DT_BF16: case DT_I16: case DT_U16: return 2;
    case DT_F32: case DT_I32: case DT_U32: return 4;
    case DT_F64: case DT_I64: case DT_U64: return 8;
    default: return 0;
  }
}
static bool mul_ok(uint64_t a, uint64_t b, uint64_t* out) { return !__builtin_mul_overflow(a, b, out); }
static bool add_ok(uint64_t a, uint64_t b, uint64_t* out) { return !__builtin_add_overflow(a, b, out); }

// element count of a shape (1 for rank 0); false on overflow
static bool shape_count(const std::vector<uint64_t>& shape, uint64_t* out) {
  uint64_t n = 1;
  for (uint64_t d : shape)
    if (!mul_ok(n, d, &n)) return false;
  *out = n;
  return true;
}

// The shape half of the destination check (fileio.rs:216-231): rank and every dimension for a tensor view, then
// the exact element count.
static int64_t check_shape(const std::vector<uint64_t>& shape, int64_t dest_len, const int64_t* dims, int64_t rank, uint64_t* count) {
  uint64_t n;
  if (!shape_count(shape, &n)) return IO_BAD_HEADER;
  if (dims) {
    bool same = (uint64_t)rank == shape.size();
    for (size_t i = 0; same && i < shape.size(); ++i) same = dims[i] >= 0 && (uint64_t)dims[i] == shape[i];
    if (!same) return IO_SHAPE_MISMATCH;
  }
  if (dest_len < 0 || (uint64_t)dest_len != n) return IO_SHAPE_MISMATCH;
  *count = n;
  return 0;
}

// ---------------------------------------------------------------------------------------------------------
// ggml's type table
// ---------------------------------------------------------------------------------------------------------
static const GgmlType kTypes[] = {
    {0, "F32", 1, 4, DT_F32, false},      {1, "F16", 1, 2, DT_F16, false},      {2, "Q4_0", 32, 18, -1, true},
    {3, "Q4_1", 32, 20, -1, true},        {6, "Q5_0", 32, 22, -1, true},        {7, "Q5_1", 32, 24, -1, true},
    {8, "Q8_0", 32, 34, -1, true},        {9, "Q8_1", 32, 36, -1, false},       {10, "Q2_K", 256, 84, -1, true},
    {11, "Q3_K", 256, 110, -1, true},     {12, "Q4_K", 256, 144, -1, true},     {13, "Q5_K", 256, 176, -1, true},
    {14, "Q6_K", 256, 210, -1, true},     {15, "Q8_K", 256, 292, -1, true},     {16, "IQ2_XXS", 256, 66, -1, false},
    {17, "IQ2_XS", 256, 74, -1, false},   {18, "IQ3_XXS", 256, 98, -1, false},  {19, "IQ1_S", 256, 50, -1, false},
    {20, "IQ4_NL", 32, 18, -1, true},     {21, "IQ3_S", 256, 110, -1, false},   {22, "IQ2_S", 256, 82, -1, false},
    {23, "IQ4_XS", 256, 136, -1, true},   {24, "I8", 1, 1, DT_I8, false},       {25, "I16", 1, 2, DT_I16, false},
    {26, "I32", 1, 4, DT_I32, false},     {27, "I64", 1, 8, DT_I64, false},     {28, "F64", 1, 8, DT_F64, false},
    {29, "IQ1_M", 256, 56, -1, false},    {30, "BF16", 1, 2, DT_BF16, false},   {34, "TQ1_0", 256, 54, -1, false},
    {35, "TQ2_0", 256, 66, -1, false},    {39, "MXFP4", 32, 17, -1, false},
};
const GgmlType* ggml_type(uint32_t id) {
  for (const GgmlType& t : kTypes)
    if (t.id == id) return &t;
  return nullptr;
}

// ---------------------------------------------------------------------------------------------------------
// a bounded little-endian reader over a FILE: every length is checked against the file before it is read, so a
// length that runs past the end is a malformed header (never a giant allocation) and only a failed read is -2
// ---------------------------------------------------------------------------------------------------------
struct Cursor {
  FILE* f;
  uint64_t pos, len;
  int64_t err = 0;

  bool need(uint64_t n) {
    if (err) return false;
    if ((len > pos ? len - pos : 0) < n) { err = IO_BAD_HEADER; return false; }
    return true;
  }
  bool fill(void* dst, uint64_t n) {
    if (!need(n)) return false;
    if (n && fread(dst, 1, n, f) != n) { err = IO_ERROR; return false; }
    pos += n;
    return true;
  }
  bool skip(uint64_t n) {
    if (!need(n)) return false;
    if (n && fseeko(f, (off_t)n, SEEK_CUR) != 0) { err = IO_ERROR; return false; }
    pos += n;
    return true;
  }
  uint32_t u32() { uint8_t b[4] = {0, 0, 0, 0}; fill(b, 4); return (uint32_t)b[0] | (uint32_t)b[1] << 8 | (uint32_t)b[2] << 16 | (uint32_t)b[3] << 24; }
  uint64_t u64() { const uint64_t lo = u32(); const uint64_t hi = u32(); return lo | hi << 32; }
  bool string(std::string* s) {
    const uint64_t n = u64();
    if (!need(n)) return false;
    s->resize((size_t)n);
    return fill(s->data(), n);
  }
};

// metadata values: the thirteen GGUF value types (gguf.rs:86-113)
enum : uint32_t { VT_U8 = 0, VT_I8, VT_U16, VT_I16, VT_U32, VT_I32, VT_F32, VT_BOOL, VT_STRING, VT_ARRAY, VT_U64, VT_I64, VT_F64 };
static const uint32_t MAX_NESTING = 64;

struct Meta {
  uint32_t type = 0;
  uint64_t bits = 0;          // the raw little-endian bits of a scalar
  std::string str;
  uint32_t elem = 0;
  std::vector<Meta> items;
};

static uint64_t fixed_size(uint32_t t) {
  switch (t) {
    case VT_U8: case VT_I8: case VT_BOOL: return 1;
    case VT_U16: case VT_I16: return 2;
    case VT_U32: case VT_I32: case VT_F32: return 4;
    case VT_U64: case VT_I64: case VT_F64: return 8;
    default: return 0;
  }
}

// Walk one value with every check; keep it in *out when out != nullptr.
static bool read_value(Cursor& c, uint32_t ty, uint32_t depth, Meta* out) {
  if (out) out->type = ty;
  if (const uint64_t sz = fixed_size(ty)) {
    uint8_t b[8] = {0};
    if (!c.fill(b, sz)) return false;
    if (out) {
      uint64_t v = 0;
      for (uint64_t i = 0; i < sz; ++i) v |= (uint64_t)b[i] << (8 * i);
      out->bits = v;
    }
    return true;
  }
  if (ty == VT_STRING) {
    if (out) return c.string(&out->str);
    const uint64_t n = c.u64();
    return c.skip(n);
  }
  if (ty != VT_ARRAY || depth >= MAX_NESTING) { if (!c.err) c.err = IO_BAD_HEADER; return false; }
  const uint32_t elem = c.u32();
  const uint64_t n = c.u64();
  if (c.err) return false;
  uint64_t min = fixed_size(elem);
  if (!min) {
    if (elem == VT_STRING) min = 8;
    else if (elem == VT_ARRAY) min = 12;
    else { c.err = IO_BAD_HEADER; return false; }
  }
  uint64_t total;
  if (!mul_ok(n, min, &total)) { c.err = IO_BAD_HEADER; return false; }
  if (!c.need(total)) return false;             // a count the rest of the file cannot hold
  if (out) { out->elem = elem; out->items.resize((size_t)n); }
  if (!out && fixed_size(elem)) return c.skip(total);
  for (uint64_t i = 0; i < n; ++i)
    if (!read_value(c, elem, depth + 1, out ? &out->items[(size_t)i] : nullptr)) return false;
  return true;
}

struct TensorInfo {
  std::string name;
  std::vector<uint64_t> ne;     // innermost first, as in the file
  uint32_t ggml_type;
  uint64_t offset;
};
struct Gguf {
  uint32_t version = 0;
  std::vector<std::pair<std::string, Meta>> metadata;
  std::vector<TensorInfo> tensors;
  uint64_t alignment = 32, data_start = 0, file_len = 0;

  const Meta* meta(const std::string& key) const {
    for (const auto& kv : metadata)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  int64_t find(const std::string& name) const {
    for (size_t i = 0; i < tensors.size(); ++i)
      if (tensors[i].name == name) return (int64_t)i;
    return -1;
  }
};

// Parse the header: magic, version, every metadata value (kept when keep_meta, else only general.alignment)
// and the whole tensor table (gguf.rs:486-578).  Returns 0 or a negative code.
static int64_t gguf_parse(FILE* f, uint64_t file_len, bool keep_meta, Gguf* g) {
  Cursor c{f, 0, file_len};
  uint8_t magic[4] = {0, 0, 0, 0};
  if (!c.fill(magic, 4)) return c.err;
  if (memcmp(magic, "GGUF", 4) != 0) return IO_BAD_HEADER;
  g->version = c.u32();
  if (c.err) return c.err;
  if (g->version < 2 || g->version > 3) return IO_BAD_HEADER;
  const uint64_t n_tensors = c.u64();
  const uint64_t n_kv = c.u64();
  if (c.err) return c.err;
  std::set<std::string> keys;
  for (uint64_t i = 0; i < n_kv; ++i) {
    std::string key;
    if (!c.string(&key)) return c.err;
    const uint32_t ty = c.u32();
    if (c.err) return c.err;
    const bool keep = keep_meta || key == "general.alignment";
    Meta v;
    if (!read_value(c, ty, 0, keep ? &v : nullptr)) return c.err ? c.err : IO_BAD_HEADER;
    if (!keys.insert(key).second) return IO_BAD_HEADER;
    if (keep) g->metadata.emplace_back(std::move(key), std::move(v));
  }
  if (const Meta* a = g->meta("general.alignment")) {
    const uint64_t v = a->bits;
    if (a->type != VT_U32 || v == 0 || (v & (v - 1)) != 0) return IO_BAD_HEADER;
    g->alignment = v;
  }
  std::set<std::string> names;
  for (uint64_t i = 0; i < n_tensors; ++i) {
    TensorInfo t;
    if (!c.string(&t.name)) return c.err;
    const uint32_t n_dims = c.u32();
    if (c.err) return c.err;
    if (n_dims > 4) return IO_BAD_HEADER;
    for (uint32_t d = 0; d < n_dims; ++d) {
      const uint64_t v = c.u64();
      if (c.err) return c.err;
      if (v > (uint64_t)INT64_MAX) return IO_BAD_HEADER;
      t.ne.push_back(v);
    }
    t.ggml_type = c.u32();
    t.offset = c.u64();
    if (c.err) return c.err;
    if (!names.insert(t.name).second) return IO_BAD_HEADER;
    g->tensors.push_back(std::move(t));
  }
  const uint64_t rem = c.pos % g->alignment;
  uint64_t start = c.pos;
  if (rem && !add_ok(c.pos, g->alignment - rem, &start)) return IO_BAD_HEADER;
  g->data_start = start;
  g->file_len = file_len;
  return 0;
}

struct File {
  FILE* f = nullptr;
  ~File() { if (f) fclose(f); }
};

// Open, size, parse: -1 if the file cannot be opened, -2 if it cannot be sized, else the parse's own result.
static int64_t gguf_open(const char* path, bool keep_meta, File* file, Gguf* g) {
  if (!path) return IO_OPEN_FAILED;
  file->f = fopen(path, "rb");
  if (!file->f) return IO_OPEN_FAILED;
  struct stat st;
  if (fstat(fileno(file->f), &st) != 0) return IO_ERROR;
  return gguf_parse(file->f, (uint64_t)st.st_size, keep_meta, g);
}

// Locate the named tensor and check it against the file (gguf.rs:623-649), then plan the move into a
// destination of dest_len elements of dest_dt (gguf.rs:678-716): type and dtype first, then dims and count.
static int64_t gguf_plan(const Gguf& g, const char* name, int64_t dest_dt, int64_t dest_len, const int64_t* dims, int64_t rank,
                         Located* out) {
  const int64_t idx = g.find(name ? name : "");
  if (idx < 0) return IO_NAME_NOT_FOUND;
  const TensorInfo& t = g.tensors[(size_t)idx];
  const GgmlType* ty = ggml_type(t.ggml_type);
  if (!ty) return IO_UNSUPPORTED_TYPE;
  uint64_t numel;
  if (!shape_count(t.ne, &numel)) return IO_BAD_HEADER;
  const uint64_t inner = t.ne.empty() ? 1 : t.ne[0];
  if (inner % ty->block != 0) return IO_BAD_HEADER;
  uint64_t nbytes, data_off, end;
  if (!mul_ok(numel / ty->block, ty->bytes, &nbytes)) return IO_BAD_HEADER;
  if (t.offset % g.alignment != 0) return IO_BAD_HEADER;
  if (!add_ok(g.data_start, t.offset, &data_off) || !add_ok(data_off, nbytes, &end) || end > g.file_len) return IO_BAD_HEADER;
  out->ggml_id = ty->id;
  out->src_dt = ty->dt;
  out->data_off = data_off;
  out->nbytes = nbytes;
  out->shape.assign(t.ne.rbegin(), t.ne.rend());
  if (ty->dt >= 0) {
    if (ty->dt == dest_dt && dtype_size(dest_dt)) out->move = Move::Verbatim;
    else if (dest_dt == DT_F32 && (ty->dt == DT_BF16 || ty->dt == DT_F16)) out->move = Move::Widen;
    else return IO_DTYPE_MISMATCH;
    return check_shape(out->shape, dest_len, dims, rank, &out->count);
  }
  if (dest_dt == DT_F32) {
    if (!ty->dequant) return IO_UNSUPPORTED_TYPE;
    out->move = Move::Dequant;
    return check_shape(out->shape, dest_len, dims, rank, &out->count);
  }
  if (dest_dt == DT_U8) {
    // raw block bytes: the storage shape is the shape with its innermost dimension as one row's byte length
    std::vector<uint64_t> storage = out->shape;
    if (!storage.empty()) storage.back() = storage.back() / ty->block * ty->bytes;
    out->move = Move::Raw;
    return check_shape(storage, dest_len, dims, rank, &out->count);
  }
  return IO_DTYPE_MISMATCH;
}

int64_t gguf_locate_for(const char* path, const char* name, int64_t dest_dt, int64_t dest_len, const int64_t* dims, int64_t rank,
                        Located* out) {
  File file;
  Gguf g;
  if (const int64_t rc = gguf_open(path, false, &file, &g)) return rc;
  return gguf_plan(g, name, dest_dt, dest_len, rank < 0 ? nullptr : dims, rank, out);
}

// ---------------------------------------------------------------------------------------------------------
// block dequantizers (host).  ggml's reference arithmetic in f32; products and sums rounded once each
// (this file is compiled without floating-point contraction).
// ---------------------------------------------------------------------------------------------------------
static const int8_t kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

static float half_at(const uint8_t* b, size_t at) { return f16_to_f32((uint16_t)(b[at] | (uint16_t)b[at + 1] << 8)); }

// 6-bit scale and min of sub-block j of the 12 packed scale bytes of Q4_K / Q5_K
static void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

void dequant_block_host(uint32_t id, const uint8_t* blk, float* y) {
  switch (id) {
    case 2: {   // Q4_0 { f16 d; u8 qs[16] }: element j in the low nibble of qs[j], j + 16 in the high
      const float d = half_at(blk, 0);
      for (int j = 0; j < 16; ++j) {
        y[j] = (float)((int)(blk[2 + j] & 0xF) - 8) * d;
        y[j + 16] = (float)((int)(blk[2 + j] >> 4) - 8) * d;
      }
      break;
    }
    case 3: {   // Q4_1 { f16 d; f16 m; u8 qs[16] }
      const float d = half_at(blk, 0), m = half_at(blk, 2);
      for (int j = 0; j < 16; ++j) {
        const float lo = (float)(blk[4 + j] & 0xF) * d, hi = (float)(blk[4 + j] >> 4) * d;
        y[j] = lo + m;
        y[j + 16] = hi + m;
      }
      break;
    }
    case 6: case 7: {   // Q5_0 { d; qh[4]; qs[16] } / Q5_1 { d; m; qh[4]; qs[16] }: bit j of qh is element j's fifth bit
      const bool affine = id == 7;
      const float d = half_at(blk, 0), m = affine ? half_at(blk, 2) : 0.0f;
      const int h = affine ? 4 : 2;
      const uint32_t qh = (uint32_t)blk[h] | (uint32_t)blk[h + 1] << 8 | (uint32_t)blk[h + 2] << 16 | (uint32_t)blk[h + 3] << 24;
      const uint8_t* qs = blk + h + 4;
      for (int j = 0; j < 16; ++j) {
        const int x0 = (int)((qs[j] & 0xFu) | (((qh >> j) << 4) & 0x10u));
        const int x1 = (int)((uint32_t)(qs[j] >> 4) | ((qh >> (j + 12)) & 0x10u));
        if (affine) {
          const float a = (float)x0 * d, b = (float)x1 * d;
          y[j] = a + m;
          y[j + 16] = b + m;
        } else {
          y[j] = (float)(x0 - 16) * d;
          y[j + 16] = (float)(x1 - 16) * d;
        }
      }
      break;
    }
    case 8: {   // Q8_0 { f16 d; i8 qs[32] }
      const float d = half_at(blk, 0);
      for (int j = 0; j < 32; ++j) y[j] = (float)(int8_t)blk[2 + j] * d;
      break;
    }
    case 10: {  // Q2_K { u8 scales[16]; u8 qs[64]; f16 d; f16 dmin }
      const float d = half_at(blk, 80), dmin = half_at(blk, 82);
      int yi = 0, is = 0;
      for (int n = 0; n < 2; ++n) {
        const uint8_t* q = blk + 16 + n * 32;
        for (int shift = 0; shift < 8; shift += 2)
          for (int h16 = 0; h16 < 2; ++h16) {
            const uint8_t sc = blk[is++];
            const float dl = d * (float)(sc & 0xF), ml = dmin * (float)(sc >> 4);
            for (int l = 0; l < 16; ++l) {
              const float p = dl * (float)((q[l + 16 * h16] >> shift) & 3);
              y[yi++] = p - ml;
            }
          }
      }
      break;
    }
    case 11: {  // Q3_K { u8 hmask[32]; u8 qs[64]; u8 scales[12]; f16 d }: a clear mask bit subtracts 4
      const uint8_t* hm = blk;
      const uint8_t* sr = blk + 96;
      const float d_all = half_at(blk, 108);
      int scales[16];
      for (int k = 0; k < 16; ++k) {
        const int low = k < 8 ? (sr[k] & 0xF) : (sr[k - 8] >> 4);
        const int high = (sr[8 + k % 4] >> (2 * (k / 4))) & 3;
        scales[k] = (low | (high << 4)) - 32;
      }
      int yi = 0, is = 0;
      uint8_t m = 1;
      for (int n = 0; n < 2; ++n) {
        const uint8_t* q = blk + 32 + n * 32;
        for (int shift = 0; shift < 8; shift += 2) {
          for (int h16 = 0; h16 < 2; ++h16) {
            const float dl = d_all * (float)scales[is++];
            for (int l = 0; l < 16; ++l) {
              const int at = l + 16 * h16;
              const int v = (int)((q[at] >> shift) & 3) - ((hm[at] & m) ? 0 : 4);
              y[yi++] = dl * (float)v;
            }
          }
          m = (uint8_t)(m << 1);
        }
      }
      break;
    }
    case 12: case 13: {  // Q4_K { d; dmin; scales[12]; qs[128] } / Q5_K { d; dmin; scales[12]; qh[32]; qs[128] }
      const bool five = id == 13;
      const float d = half_at(blk, 0), dmin = half_at(blk, 2);
      const uint8_t* scales = blk + 4;
      const uint8_t* qh = blk + 16;
      const uint8_t* qs = blk + (five ? 48 : 16);
      int yi = 0;
      for (int c = 0; c < 4; ++c) {
        const uint8_t* q = qs + c * 32;
        uint8_t sc1, mn1, sc2, mn2;
        scale_min_k4(2 * c, scales, &sc1, &mn1);
        scale_min_k4(2 * c + 1, scales, &sc2, &mn2);
        const float d1 = d * (float)sc1, m1 = dmin * (float)mn1, d2 = d * (float)sc2, m2 = dmin * (float)mn2;
        const uint8_t u1 = (uint8_t)(1u << (2 * c)), u2 = (uint8_t)(2u << (2 * c));
        for (int l = 0; l < 32; ++l) {
          const float p = d1 * (float)((q[l] & 0xF) + ((five && (qh[l] & u1)) ? 16 : 0));
          y[yi++] = p - m1;
        }
        for (int l = 0; l < 32; ++l) {
          const float p = d2 * (float)((q[l] >> 4) + ((five && (qh[l] & u2)) ? 16 : 0));
          y[yi++] = p - m2;
        }
      }
      break;
    }
    case 14: {  // Q6_K { u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d }
      const float d = half_at(blk, 208);
      for (int n = 0; n < 2; ++n) {
        const uint8_t* ql = blk + n * 64;
        const uint8_t* qh = blk + 128 + n * 32;
        const int8_t* sc = (const int8_t*)(blk + 192 + n * 8);
        float* yo = y + n * 128;
        for (int l = 0; l < 32; ++l) {
          const int is = l / 16;
          const int q1 = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
          const int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
          const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
          const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
          const float s0 = d * (float)sc[is], s2 = d * (float)sc[is + 2], s4 = d * (float)sc[is + 4], s6 = d * (float)sc[is + 6];
          yo[l] = s0 * (float)q1;
          yo[l + 32] = s2 * (float)q2;
          yo[l + 64] = s4 * (float)q3;
          yo[l + 96] = s6 * (float)q4;
        }
      }
      break;
    }
    case 15: {  // Q8_K { f32 d; i8 qs[256]; i16 bsums[16] }
      uint32_t u = (uint32_t)blk[0] | (uint32_t)blk[1] << 8 | (uint32_t)blk[2] << 16 | (uint32_t)blk[3] << 24;
      const float d = f32_from_bits(u);
      for (int j = 0; j < 256; ++j) y[j] = d * (float)(int8_t)blk[4 + j];
      break;
    }
    case 20: {  // IQ4_NL { f16 d; u8 qs[16] }: nibbles index the non-uniform levels
      const float d = half_at(blk, 0);
      for (int j = 0; j < 16; ++j) {
        y[j] = d * (float)kIq4nl[blk[2 + j] & 0xF];
        y[j + 16] = d * (float)kIq4nl[blk[2 + j] >> 4];
      }
      break;
    }
    case 23: {  // IQ4_XS { f16 d; u16 scales_h; u8 scales_l[4]; u8 qs[128] }
      const float d = half_at(blk, 0);
      const uint32_t scales_h = (uint32_t)blk[2] | (uint32_t)blk[3] << 8;
      for (int ib = 0; ib < 8; ++ib) {
        const int lo = (blk[4 + ib / 2] >> (4 * (ib % 2))) & 0xF;
        const int hi = (int)((scales_h >> (2 * ib)) & 3);
        const float dl = d * (float)((lo | (hi << 4)) - 32);
        const uint8_t* q = blk + 8 + ib * 16;
        for (int j = 0; j < 16; ++j) {
          y[ib * 32 + j] = dl * (float)kIq4nl[q[j] & 0xF];
          y[ib * 32 + j + 16] = dl * (float)kIq4nl[q[j] >> 4];
        }
      }
      break;
    }
    default:
      break;
  }
}

// ---------------------------------------------------------------------------------------------------------
// moving a located payload into host memory
// ---------------------------------------------------------------------------------------------------------
static const size_t STAGE_UNITS = 1 << 12;    // blocks (or half elements) per staged chunk

static int64_t transfer_host(FILE* f, const Located& loc, uint8_t* out) {
  if (loc.count == 0) return 0;
  if (fseeko(f, (off_t)loc.data_off, SEEK_SET) != 0) return IO_ERROR;
  switch (loc.move) {
    case Move::Verbatim: case Move::Raw: {
      const uint64_t bytes = loc.move == Move::Raw ? loc.count : loc.count * (uint64_t)dtype_size(loc.src_dt);
      return fread(out, 1, bytes, f) == bytes ? 0 : (int64_t)IO_ERROR;
    }
    case Move::Widen: {
      std::vector<uint8_t> stage(std::min<uint64_t>(loc.count, STAGE_UNITS) * 2);
      float* dst = reinterpret_cast<float*>(out);
      for (uint64_t done = 0; done < loc.count;) {
        const uint64_t m = std::min<uint64_t>(loc.count - done, STAGE_UNITS);
        if (fread(stage.data(), 2, m, f) != m) return IO_ERROR;
        for (uint64_t j = 0; j < m; ++j)
          dst[done + j] = widen_half_host((uint16_t)(stage[2 * j] | (uint16_t)stage[2 * j + 1] << 8), loc.src_dt);
        done += m;
      }
      return 0;
    }
    case Move::Dequant: {
      const GgmlType* ty = ggml_type(loc.ggml_id);
      const uint64_t blocks = loc.count / ty->block;
      std::vector<uint8_t> stage(std::min<uint64_t>(blocks, STAGE_UNITS) * ty->bytes);
      float* dst = reinterpret_cast<float*>(out);
      for (uint64_t done = 0; done < blocks;) {
        const uint64_t m = std::min<uint64_t>(blocks - done, STAGE_UNITS);
        if (fread(stage.data(), ty->bytes, m, f) != m) return IO_ERROR;
        for (uint64_t j = 0; j < m; ++j) dequant_block_host(ty->id, stage.data() + j * ty->bytes, dst + (done + j) * ty->block);
        done += m;
      }
      return 0;
    }
  }
  return IO_ERROR;
}

// Value i of a metadata entry: element i of an array, or the value itself when i == 0 (gguf.rs:929-937).
static int64_t meta_elem(const Gguf& g, const char* key, int64_t i, const Meta** out) {
  const Meta* v = g.meta(key ? key : "");
  if (!v) return IO_NAME_NOT_FOUND;
  if (i < 0) return IO_SHAPE_MISMATCH;
  if (v->type == VT_ARRAY) {
    if ((uint64_t)i >= v->items.size()) return IO_SHAPE_MISMATCH;
    *out = &v->items[(size_t)i];
    return 0;
  }
  if (i != 0) return IO_SHAPE_MISMATCH;
  *out = v;
  return 0;
}
static bool meta_as_i64(const Meta& v, int64_t* out) {
  switch (v.type) {
    case VT_U8: *out = (uint8_t)v.bits; return true;
    case VT_I8: *out = (int8_t)v.bits; return true;
    case VT_U16: *out = (uint16_t)v.bits; return true;
    case VT_I16: *out = (int16_t)v.bits; return true;
    case VT_U32: *out = (uint32_t)v.bits; return true;
    case VT_I32: *out = (int32_t)v.bits; return true;
    case VT_U64: case VT_I64: *out = (int64_t)v.bits; return true;
    case VT_BOOL: *out = (v.bits & 0xFF) != 0; return true;
    default: return false;
  }
}
static bool meta_as_f64(const Meta& v, double* out) {
  int64_t i;
  switch (v.type) {
    case VT_F32: *out = (double)f32_from_bits((uint32_t)v.bits); return true;
    case VT_F64: memcpy(out, &v.bits, 8); return true;
    case VT_U64: *out = (double)v.bits; return true;
    case VT_BOOL: return false;
    default:
      if (!meta_as_i64(v, &i)) return false;
      *out = (double)i;
      return true;
  }
}

// ---------------------------------------------------------------------------------------------------------
// safetensors: 8-byte little-endian header length, that many bytes of JSON, then one byte buffer
// ---------------------------------------------------------------------------------------------------------
static const uint64_t ST_MAX_HEADER = 100000000ull;
static const uint32_t ST_MAX_DEPTH = 64;

struct Json {
  enum Kind { Literal, Num, Str, Arr, Obj } kind = Literal;
  bool has_u64 = false;       // Num: a plain non-negative integer that fits u64
  uint64_t u = 0;
  std::string s;
  std::vector<Json> items;                              // Arr
  std::vector<std::pair<std::string, Json>> members;   // Obj, in source order, duplicates kept
};

// A strict recursive-descent parser of the JSON grammar (safetensors.rs:66-292 states the accepted language:
// RFC 8259 values, escapes with surrogate pairs, no control characters in strings, nesting at most 64 deep).
struct JsonParser {
  const uint8_t* b;
  size_t n, i = 0;
  uint32_t depth = 0;

  void ws() { while (i < n && (b[i] == ' ' || b[i] == '\t' || b[i] == '\n' || b[i] == '\r')) ++i; }
  bool eat(uint8_t c) { ws(); if (i < n && b[i] == c) { ++i; return true; } return false; }
  bool literal(const char* w, Json* out) {
    const size_t k = strlen(w);
    if (n - i < k || memcmp(b + i, w, k) != 0) return false;
    i += k;
    out->kind = Json::Literal;
    return true;
  }
  bool hex4(uint32_t* out) {
    if (n - i < 4) return false;
    uint32_t v = 0;
    for (int k = 0; k < 4; ++k) {
      const uint8_t d = b[i + k];
      uint32_t x;
      if (d >= '0' && d <= '9') x = d - '0';
      else if (d >= 'a' && d <= 'f') x = d - 'a' + 10;
      else if (d >= 'A' && d <= 'F') x = d - 'A' + 10;
      else return false;
      v = v * 16 + x;
    }
    i += 4;
    *out = v;
    return true;
  }
  static void utf8(uint32_t c, std::string* s) {
    if (c < 0x80) s->push_back((char)c);
    else if (c < 0x800) { s->push_back((char)(0xC0 | c >> 6)); s->push_back((char)(0x80 | (c & 0x3F))); }
    else if (c < 0x10000) { s->push_back((char)(0xE0 | c >> 12)); s->push_back((char)(0x80 | ((c >> 6) & 0x3F))); s->push_back((char)(0x80 | (c & 0x3F))); }
    else { s->push_back((char)(0xF0 | c >> 18)); s->push_back((char)(0x80 | ((c >> 12) & 0x3F))); s->push_back((char)(0x80 | ((c >> 6) & 0x3F))); s->push_back((char)(0x80 | (c & 0x3F))); }
  }
  static bool valid_utf8(const std::string& s) {
    const uint8_t* p = (const uint8_t*)s.data();
    const size_t m = s.size();
    for (size_t k = 0; k < m;) {
      const uint8_t c = p[k];
      int len;
      uint32_t cp;
      if (c < 0x80) { ++k; continue; }
      else if ((c & 0xE0) == 0xC0) { len = 2; cp = c & 0x1F; }
      else if ((c & 0xF0) == 0xE0) { len = 3; cp = c & 0x0F; }
      else if ((c & 0xF8) == 0xF0) { len = 4; cp = c & 0x07; }
      else return false;
      if (m - k < (size_t)len) return false;
      for (int t = 1; t < len; ++t) {
        if ((p[k + t] & 0xC0) != 0x80) return false;
        cp = cp << 6 | (p[k + t] & 0x3F);
      }
      if ((len == 2 && cp < 0x80) || (len == 3 && cp < 0x800) || (len == 4 && cp < 0x10000) || cp > 0x10FFFF ||
          (cp >= 0xD800 && cp < 0xE000))
        return false;
      k += len;
    }
    return true;
  }
  bool string(std::string* out) {
    if (i >= n || b[i] != '"') return false;
    ++i;
    out->clear();
    for (;;) {
      if (i >= n) return false;
      const uint8_t c = b[i++];
      if (c == '"') return valid_utf8(*out);
      if (c == '\\') {
        if (i >= n) return false;
        const uint8_t e = b[i++];
        switch (e) {
          case '"': out->push_back('"'); break;
          case '\\': out->push_back('\\'); break;
          case '/': out->push_back('/'); break;
          case 'b': out->push_back('\b'); break;
          case 'f': out->push_back('\f'); break;
          case 'n': out->push_back('\n'); break;
          case 'r': out->push_back('\r'); break;
          case 't': out->push_back('\t'); break;
          case 'u': {
            uint32_t hi, code;
            if (!hex4(&hi)) return false;
            if (hi >= 0xD800 && hi < 0xDC00) {
              uint32_t lo;
              if (n - i < 2 || b[i] != '\\' || b[i + 1] != 'u') return false;
              i += 2;
              if (!hex4(&lo) || lo < 0xDC00 || lo >= 0xE000) return false;
              code = 0x10000 + ((hi - 0xD800) << 10) + (lo - 0xDC00);
            } else {
              if (hi >= 0xDC00 && hi < 0xE000) return false;    // a lone low surrogate is not a character
              code = hi;
            }
            utf8(code, out);
            break;
          }
          default: return false;
        }
      } else if (c < 0x20) {
        return false;
      } else {
        out->push_back((char)c);
      }
    }
  }
  bool digits() { const size_t s = i; while (i < n && b[i] >= '0' && b[i] <= '9') ++i; return i > s; }
  bool number(Json* out) {
    const bool neg = i < n && b[i] == '-';
    if (neg) ++i;
    const size_t int_start = i;
    if (i >= n) return false;
    if (b[i] == '0') ++i;
    else if (b[i] >= '1' && b[i] <= '9') { while (i < n && b[i] >= '0' && b[i] <= '9') ++i; }
    else return false;
    const size_t int_end = i;
    bool plain = !neg;
    if (i < n && b[i] == '.') { plain = false; ++i; if (!digits()) return false; }
    if (i < n && (b[i] == 'e' || b[i] == 'E')) {
      plain = false;
      ++i;
      if (i < n && (b[i] == '+' || b[i] == '-')) ++i;
      if (!digits()) return false;
    }
    out->kind = Json::Num;
    out->has_u64 = false;
    if (plain) {
      uint64_t v = 0;
      bool fits = true;
      for (size_t k = int_start; k < int_end && fits; ++k) fits = mul_ok(v, 10, &v) && add_ok(v, (uint64_t)(b[k] - '0'), &v);
      out->has_u64 = fits;
      out->u = v;
    }
    return true;
  }
  bool value(Json* out) {
    ws();
    if (i >= n) return false;
    switch (b[i]) {
      case '{': case '[': {
        if (depth >= ST_MAX_DEPTH) return false;
        ++depth;
        const bool ok = b[i] == '{' ? object(out) : array(out);
        --depth;
        return ok;
      }
      case '"': out->kind = Json::Str; return string(&out->s);
      case 't': return literal("true", out);
      case 'f': return literal("false", out);
      case 'n': return literal("null", out);
      default:
        if (b[i] == '-' || (b[i] >= '0' && b[i] <= '9')) return number(out);
        return false;
    }
  }
  bool object(Json* out) {
    out->kind = Json::Obj;
    if (!eat('{')) return false;
    if (eat('}')) return true;
    for (;;) {
      ws();
      std::string key;
      if (!string(&key)) return false;
      if (!eat(':')) return false;
      Json v;
      if (!value(&v)) return false;
      out->members.emplace_back(std::move(key), std::move(v));
      if (eat(',')) continue;
      return eat('}');
    }
  }
  bool array(Json* out) {
    out->kind = Json::Arr;
    if (!eat('[')) return false;
    if (eat(']')) return true;
    for (;;) {
      Json v;
      if (!value(&v)) return false;
      out->items.push_back(std::move(v));
      if (eat(',')) continue;
      return eat(']');
    }
  }
};

static int64_t st_dtype(const std::string& s) {
  static const struct { const char* n; int64_t dt; } table[] = {
      {"F32", DT_F32}, {"F64", DT_F64}, {"F16", DT_F16}, {"BF16", DT_BF16}, {"I8", DT_I8}, {"I16", DT_I16},
      {"I32", DT_I32}, {"I64", DT_I64}, {"U8", DT_U8},   {"U16", DT_U16},   {"U32", DT_U32}, {"U64", DT_U64}};
  for (const auto& e : table)
    if (s == e.n) return e.dt;
  return DT_UNSUPPORTED;
}
static const Json* member(const Json& obj, const char* key) {
  for (const auto& m : obj.members)
    if (m.first == key) return &m.second;
  return nullptr;
}
static bool u64_list(const Json* v, std::vector<uint64_t>* out) {
  if (!v || v->kind != Json::Arr) return false;
  for (const Json& x : v->items) {
    if (x.kind != Json::Num || !x.has_u64) return false;
    out->push_back(x.u);
  }
  return true;
}

// Locate `name`: parse the header, find the entry, map its dtype, check its extent against the file and its
// byte length against dtype x shape (safetensors.rs:308-367, fileio.rs:167-181); then the destination check.
static int64_t st_plan(FILE* f, uint64_t file_len, const char* name_c, int64_t dest_dt, int64_t dest_len, const int64_t* dims,
                       int64_t rank, Located* out) {
  if (file_len < 8) return IO_BAD_HEADER;
  uint8_t le[8];
  if (fseeko(f, 0, SEEK_SET) != 0 || fread(le, 1, 8, f) != 8) return IO_ERROR;
  uint64_t hlen = 0;
  for (int k = 0; k < 8; ++k) hlen |= (uint64_t)le[k] << (8 * k);
  if (hlen > ST_MAX_HEADER || hlen > file_len - 8) return IO_BAD_HEADER;
  std::vector<uint8_t> header((size_t)hlen);
  if (hlen && fread(header.data(), 1, hlen, f) != hlen) return IO_ERROR;
  JsonParser p{header.data(), header.size()};
  Json root;
  if (!p.value(&root)) return IO_BAD_HEADER;
  p.ws();
  if (p.i != p.n || root.kind != Json::Obj) return IO_BAD_HEADER;
  const std::string name = name_c ? name_c : "";
  if (name == "__metadata__") return IO_NAME_NOT_FOUND;
  const Json* entry = nullptr;
  for (const auto& m : root.members)
    if (m.first == name) {
      if (entry) return IO_BAD_HEADER;         // a name that occurs twice
      entry = &m.second;
    }
  if (!entry) return IO_NAME_NOT_FOUND;
  if (entry->kind != Json::Obj) return IO_BAD_HEADER;
  const Json* dt = member(*entry, "dtype");
  if (!dt || dt->kind != Json::Str) return IO_BAD_HEADER;
  const int64_t dtype = st_dtype(dt->s);
  std::vector<uint64_t> shape, offsets;
  if (!u64_list(member(*entry, "shape"), &shape)) return IO_BAD_HEADER;
  if (!u64_list(member(*entry, "data_offsets"), &offsets) || offsets.size() != 2) return IO_BAD_HEADER;
  const uint64_t begin = offsets[0], end = offsets[1];
  if (begin > end) return IO_BAD_HEADER;
  uint64_t data_off, last;
  if (!add_ok(8 + hlen, begin, &data_off)) return IO_BAD_HEADER;
  const uint64_t nbytes = end - begin;
  if (!add_ok(data_off, nbytes, &last) || last > file_len) return IO_BAD_HEADER;
  if (const int64_t sz = dtype_size(dtype)) {
    uint64_t n, want;
    if (!shape_count(shape, &n) || !mul_ok(n, (uint64_t)sz, &want) || want != nbytes) return IO_BAD_HEADER;
  }
  out->src_dt = dtype;
  out->data_off = data_off;
  out->nbytes = nbytes;
  out->shape = shape;
  if (dtype == dest_dt && dtype_size(dest_dt)) out->move = Move::Verbatim;
  else if (dest_dt == DT_F32 && (dtype == DT_BF16 || dtype == DT_F16)) out->move = Move::Widen;
  else return IO_DTYPE_MISMATCH;
  return check_shape(shape, dest_len, dims, rank, &out->count);
}

static int64_t st_open(const char* path, File* file, uint64_t* file_len) {
  if (!path) return IO_OPEN_FAILED;
  file->f = fopen(path, "rb");
  if (!file->f) return IO_OPEN_FAILED;
  struct stat st;
  if (fstat(fileno(file->f), &st) != 0) return IO_ERROR;
  *file_len = (uint64_t)st.st_size;
  return 0;
}

int64_t st_locate_for(const char* path, const char* name, int64_t dest_dt, int64_t dest_len, const int64_t* dims, int64_t rank,
                      Located* out) {
  File file;
  uint64_t file_len = 0;
  if (const int64_t rc = st_open(path, &file, &file_len)) return rc;
  return st_plan(file.f, file_len, name, dest_dt, dest_len, rank < 0 ? nullptr : dims, rank, out);
}

}  // namespace wkb_io

using namespace wkb_io;

extern "C" {

// gguf_read_<T>(path, name, buf): the element count, or -1 (open), -2 (I/O), -3 (dtype), -4 (shape or count),
// -5 (no such name), -6 (malformed header), -7 (a type with no decoder).  rank < 0: a flat destination.
int64_t wukong_rt_gguf_read(const char* path, const char* name, void* data, int64_t len, int64_t dtype, const int64_t* dims,
                            int64_t rank) {
  File file;
  Gguf g;
  if (const int64_t rc = gguf_open(path, false, &file, &g)) return rc;
  Located loc;
  if (const int64_t rc = gguf_plan(g, name, dtype, len, rank < 0 ? nullptr : dims, rank, &loc)) return rc;
  if (const int64_t rc = transfer_host(file.f, loc, static_cast<uint8_t*>(data))) return rc;
  return (int64_t)loc.count;
}

// gguf_find / gguf_rank / gguf_dim / gguf_type (what = 0..3): the answer, -5 for no such tensor, -4 for a
// dimension index outside 0..rank, -2 for an unknown query.
int64_t wukong_rt_gguf_query(const char* path, const char* name, int64_t what, int64_t k) {
  File file;
  Gguf g;
  if (const int64_t rc = gguf_open(path, false, &file, &g)) return rc;
  const int64_t i = g.find(name ? name : "");
  if (i < 0) return IO_NAME_NOT_FOUND;
  const TensorInfo& t = g.tensors[(size_t)i];
  switch (what) {
    case 0: return i;
    case 1: return (int64_t)t.ne.size();
    case 2: return (k >= 0 && (uint64_t)k < t.ne.size()) ? (int64_t)t.ne[t.ne.size() - 1 - (size_t)k] : IO_SHAPE_MISMATCH;
    case 3: return (int64_t)t.ggml_type;
    default: return IO_ERROR;
  }
}

// gguf_meta_type / gguf_meta_len / gguf_meta_i64 (what = 0..2).  The two queries report -5 for a missing key and
// the file's own code for a bad file; the value read reports nothing but its default.
int64_t wukong_rt_gguf_meta(const char* path, const char* key, int64_t what, int64_t i, int64_t dflt) {
  File file;
  Gguf g;
  if (const int64_t rc = gguf_open(path, true, &file, &g)) return what == 2 ? dflt : rc;
  switch (what) {
    case 0: { const Meta* v = g.meta(key ? key : ""); return v ? (int64_t)v->type : IO_NAME_NOT_FOUND; }
    case 1: {
      const Meta* v = g.meta(key ? key : "");
      if (!v) return IO_NAME_NOT_FOUND;
      return v->type == VT_STRING ? (int64_t)v->str.size() : v->type == VT_ARRAY ? (int64_t)v->items.size() : 1;
    }
    case 2: {
      const Meta* v = nullptr;
      int64_t out;
      return (meta_elem(g, key, i, &v) == 0 && meta_as_i64(*v, &out)) ? out : dflt;
    }
    default: return IO_ERROR;
  }
}

double wukong_rt_gguf_meta_f64(const char* path, const char* key, int64_t i, double dflt) {
  File file;
  Gguf g;
  if (gguf_open(path, true, &file, &g)) return dflt;
  const Meta* v = nullptr;
  double out;
  return (meta_elem(g, key, i, &v) == 0 && meta_as_f64(*v, &out)) ? out : dflt;
}

// gguf_meta_str: copy string value i into buf as snprintf does (at most len - 1 bytes, then a NUL; nothing for
// len <= 0) and return its full byte length, or a negative code (-3: not a string) with buf untouched.
int64_t wukong_rt_gguf_meta_str(const char* path, const char* key, int64_t i, char* buf, int64_t len) {
  File file;
  Gguf g;
  if (const int64_t rc = gguf_open(path, true, &file, &g)) return rc;
  const Meta* v = nullptr;
  if (const int64_t rc = meta_elem(g, key, i, &v)) return rc;
  if (v->type != VT_STRING) return IO_DTYPE_MISMATCH;
  if (len > 0 && buf) {
    const size_t n = std::min<size_t>(v->str.size(), (size_t)len - 1);
    memcpy(buf, v->str.data(), n);
    buf[n] = 0;
  }
  return (int64_t)v->str.size();
}

// st_read_<T>(path, name, buf): verbatim, or f32 widened from a BF16 / F16 payload; codes as above (no -7).
int64_t wukong_rt_st_read(const char* path, const char* name, void* data, int64_t len, int64_t dtype, const int64_t* dims,
                          int64_t rank) {
  File file;
  uint64_t file_len = 0;
  if (const int64_t rc = st_open(path, &file, &file_len)) return rc;
  Located loc;
  if (const int64_t rc = st_plan(file.f, file_len, name, dtype, len, rank < 0 ? nullptr : dims, rank, &loc)) return rc;
  if (const int64_t rc = transfer_host(file.f, loc, static_cast<uint8_t*>(data))) return rc;
  return (int64_t)loc.count;
}

}  // extern "C"
