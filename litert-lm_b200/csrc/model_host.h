// Host-side model ingestion: `.litertlm` container walk, weights-record index,
// and the repacks from the canonical int4 layout into the two device layouts.
// No CUDA in this header; everything here is unit-tested on CPU.
#pragma once
#include <stdint.h>
#include <string.h>

#include <cmath>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"

namespace b200lm {

// ------------------------------------------------------------ `.litertlm`
// Layout (reference: schema/core/litertlm_export.cc:126-173,
// schema/core/litertlm_read.cc:38-109): "LITERTLM", u32 major/minor/patch,
// 4 pad bytes, u64 header end, flatbuffer LiteRTLMMetaData at byte 32, sections
// on 16 KiB boundaries.

struct SectionRef {
  int data_type;
  uint64_t begin, end;
};

class FlatView {
 public:
  FlatView(const uint8_t* b, size_t n) : b_(b), n_(n) {}
  bool ok(size_t p, size_t len) const { return p + len <= n_ && p + len >= p; }
  uint32_t u32(size_t p) const { uint32_t v = 0; if (ok(p, 4)) memcpy(&v, b_ + p, 4); else bad_ = true; return v; }
  int32_t i32(size_t p) const { return (int32_t)u32(p); }
  uint16_t u16(size_t p) const { uint16_t v = 0; if (ok(p, 2)) memcpy(&v, b_ + p, 2); else bad_ = true; return v; }
  uint64_t u64(size_t p) const { uint64_t v = 0; if (ok(p, 8)) memcpy(&v, b_ + p, 8); else bad_ = true; return v; }
  uint8_t u8(size_t p) const { if (!ok(p, 1)) { bad_ = true; return 0; } return b_[p]; }
  size_t indirect(size_t p) const { return p + u32(p); }
  // position of field `idx` inside table at tpos, 0 when absent
  size_t field(size_t tpos, int idx) const {
    size_t vt = tpos - (size_t)(int64_t)i32(tpos);
    uint16_t vsz = u16(vt);
    size_t slot = 4 + 2 * (size_t)idx;
    if (slot >= vsz) return 0;
    uint16_t o = u16(vt + slot);
    return o ? tpos + o : 0;
  }
  bool bad() const { return bad_; }

 private:
  const uint8_t* b_;
  size_t n_;
  mutable bool bad_ = false;
};

inline std::vector<SectionRef> parse_litertlm_sections(const uint8_t* data, size_t n) {
  B2_CHECK(n >= 32 && memcmp(data, "LITERTLM", 8) == 0, kInvalidArgument,
           "Invalid magic number or failed to read");
  uint32_t major;
  memcpy(&major, data + 8, 4);
  B2_CHECK(major == 1, kUnimplemented, "This reader doesn't support version " + std::to_string(major) +
                                           ", expected version 1.");
  uint64_t header_end;
  memcpy(&header_end, data + 24, 8);
  B2_CHECK(header_end >= 32, kInvalidArgument, "Invalid header end offset: smaller than current position.");
  B2_CHECK(header_end <= n, kInternal, "Failed to read header data.");
  FlatView f(data + 32, (size_t)(header_end - 32));
  std::vector<SectionRef> out;
  size_t root = f.indirect(0);
  size_t smf = f.field(root, 1);
  B2_CHECK(smf != 0 && !f.bad(), kInvalidArgument, "header has no section metadata");
  size_t sm = f.indirect(smf);
  size_t vecf = f.field(sm, 0);
  B2_CHECK(vecf != 0 && !f.bad(), kInvalidArgument, "section metadata has no objects");
  size_t vec = f.indirect(vecf);
  uint32_t count = f.u32(vec);
  B2_CHECK(!f.bad() && count < 4096, kInvalidArgument, "corrupt section vector");
  for (uint32_t i = 0; i < count; ++i) {
    size_t so = f.indirect(vec + 4 + 4 * (size_t)i);
    SectionRef s{0, 0, 0};
    size_t bf = f.field(so, 1), ef = f.field(so, 2), tf = f.field(so, 3);
    if (bf) s.begin = f.u64(bf);
    if (ef) s.end = f.u64(ef);
    if (tf) s.data_type = f.u8(tf);
    B2_CHECK(!f.bad(), kInvalidArgument, "corrupt section object");
    B2_CHECK(s.begin <= s.end && s.end <= n, kInvalidArgument, "section range outside the file (truncated?)");
    out.push_back(s);
  }
  return out;
}

// ------------------------------------------------------------ weights record

struct TensorEntry {
  char name[48];
  uint32_t dtype, rows, cols, pad;
  uint64_t offset, nbytes;
};
static_assert(sizeof(TensorEntry) == 80, "index entry is 80 bytes");

struct WeightsRecord {
  const uint8_t* base = nullptr;
  size_t size = 0;
  ModelDims dims{};
  uint32_t n_tensors = 0;
  const TensorEntry* find(const std::string& name) const {
    const TensorEntry* e = reinterpret_cast<const TensorEntry*>(base + 256);
    for (uint32_t i = 0; i < n_tensors; ++i)
      if (strncmp(e[i].name, name.c_str(), 48) == 0) return &e[i];
    return nullptr;
  }
  const TensorEntry& need(const std::string& name, uint32_t dtype) const {
    const TensorEntry* e = find(name);
    B2_CHECK(e != nullptr, kNotFound, "tensor missing from weights record: " + name);
    B2_CHECK(e->dtype == dtype, kInvalidArgument, "tensor has the wrong type: " + name);
    B2_CHECK(e->offset + e->nbytes <= size, kInvalidArgument, "tensor data outside the record: " + name);
    return *e;
  }
};

inline WeightsRecord open_weights_record(const uint8_t* p, size_t n) {
  B2_CHECK(n >= 512 && memcmp(p, "B2LMWT01", 8) == 0, kInvalidArgument, "not a weights record");
  WeightsRecord r;
  r.base = p;
  r.size = n;
  memcpy(&r.n_tensors, p + 12, 4);
  B2_CHECK(256 + (size_t)r.n_tensors * sizeof(TensorEntry) <= n, kInvalidArgument, "weights record index truncated");
  int32_t ic[16];
  float fc[8];
  int32_t bk[8];
  memcpy(ic, p + 16, sizeof ic);
  memcpy(fc, p + 80, sizeof fc);
  memcpy(bk, p + 112, sizeof bk);
  ModelDims& d = r.dims;
  d.n_layers = ic[0]; d.d = ic[1]; d.hq = ic[2]; d.hkv = ic[3]; d.hd = ic[4]; d.ffn = ic[5];
  d.vocab = ic[6]; d.max_ctx = ic[7]; d.window = ic[8]; d.period = ic[9]; d.kv_dtype = ic[10];
  d.n_buckets = ic[11];
  B2_CHECK(d.n_buckets >= 1 && d.n_buckets <= kMaxBuckets, kInvalidArgument, "bad prefill bucket count");
  for (int i = 0; i < d.n_buckets; ++i) d.buckets[i] = bk[i];
  for (int i = 1; i < d.n_buckets; ++i)
    B2_CHECK(d.buckets[i] < d.buckets[i - 1] && d.buckets[i] > 0, kInvalidArgument, "buckets must descend");
  d.rope_local = fc[0]; d.rope_global = fc[1]; d.eps = fc[2];
  B2_CHECK(d.n_layers > 0 && d.d > 0 && d.hq > 0 && d.hkv > 0 && d.period > 0, kInvalidArgument, "bad model shape");
  B2_CHECK(d.hq % d.hkv == 0, kInvalidArgument, "query heads must be a multiple of kv heads");
  int G = d.hq / d.hkv;
  B2_CHECK(G == 1 || G == 2 || G == 4, kUnimplemented, "GQA group size must be 1, 2 or 4");
  B2_CHECK(d.hd == 32 || d.hd == 64 || d.hd == 128 || d.hd == 256, kUnimplemented, "head_dim must be 32/64/128/256");
  B2_CHECK(d.d % 64 == 0 && d.ffn % 64 == 0 && (d.hq * d.hd) % 64 == 0, kUnimplemented,
           "d_model, ffn and q width must be multiples of 64");
  B2_CHECK(d.vocab % 16 == 0 && d.nqkv() % 16 == 0, kUnimplemented, "row counts must be multiples of 16");
  B2_CHECK(d.kv_dtype == 0 || d.kv_dtype == 1, kInvalidArgument, "kv dtype must be 0 (fp32) or 1 (bf16)");
  return r;
}

// Finds the weights record inside a `.litertlm` image (GenericBinaryData
// section, type 1, that starts with the record magic) or accepts a bare record.
inline WeightsRecord locate_weights(const uint8_t* data, size_t n) {
  if (n >= 8 && memcmp(data, "B2LMWT01", 8) == 0) return open_weights_record(data, n);
  auto secs = parse_litertlm_sections(data, n);
  for (const auto& s : secs)
    if (s.data_type == 1 && s.end - s.begin >= 512 && memcmp(data + s.begin, "B2LMWT01", 8) == 0)
      return open_weights_record(data + s.begin, (size_t)(s.end - s.begin));
  throw Error{kNotFound, "no int4 decoder weights record in the .litertlm file"};
}

// ------------------------------------------------------------ repacks

inline int canon_q(const uint8_t* packed, int64_t K, int64_t row, int64_t k) {
  uint8_t b = packed[row * (K / 2) + (k >> 1)];
  int nib = (k & 1) ? (b >> 4) : (b & 0xF);
  return nib >= 8 ? nib - 16 : nib;
}

template <typename F>
inline void parallel_for(int64_t n, F fn) {
  unsigned nt = std::thread::hardware_concurrency();
  if (nt == 0) nt = 4;
  if (nt > 32) nt = 32;
  if (n < 64) nt = 1;
  std::vector<std::thread> th;
  int64_t per = (n + nt - 1) / nt;
  for (unsigned t = 0; t < nt; ++t) {
    int64_t a = t * per, b = std::min<int64_t>(n, a + per);
    if (a >= b) break;
    th.emplace_back([=] { for (int64_t i = a; i < b; ++i) fn(i); });
  }
  for (auto& x : th) x.join();
}

// mma-tiled layout ("W4T"): 16x64 tiles of 512 bytes ordered [row_tile][k_tile];
// lane l = 4g + t owns words 0..3; word j covers k = 32*(j/2) + 16*(j%2) + 4t + i,
// nibble 2i = row g, nibble 2i+1 = row g + 8, two's complement.
// row_map(tile_row) gives the source row of each destination row (used to
// interleave gate and up tiles); rows < 0 are zero rows.
template <typename RowMap>
inline void repack_w4t(const uint8_t* packed, int64_t n_dst_rows, int64_t K, RowMap row_map, uint32_t* out) {
  const int64_t KT = K / 64, RT = n_dst_rows / 16;
  parallel_for(RT, [&](int64_t rt) {
    for (int64_t kt = 0; kt < KT; ++kt) {
      uint32_t* blk = out + (rt * KT + kt) * 128;
      for (int l = 0; l < 32; ++l) {
        int g = l >> 2, t = l & 3;
        int64_t r0 = row_map(rt * 16 + g), r1 = row_map(rt * 16 + g + 8);
        for (int j = 0; j < 4; ++j) {
          int64_t kq = kt * 64 + 32 * (j >> 1) + 16 * (j & 1) + 4 * t;
          uint32_t w = 0;
          for (int i = 0; i < 4; ++i) {
            uint32_t a = (uint32_t)(r0 >= 0 ? canon_q(packed, K, r0, kq + i) : 0) & 0xFu;
            uint32_t b = (uint32_t)(r1 >= 0 ? canon_q(packed, K, r1, kq + i) : 0) & 0xFu;
            w |= a << (8 * i);
            w |= b << (8 * i + 4);
          }
          blk[l * 4 + j] = w;
        }
      }
    }
  });
}

// tensor-core GEMM layout ("W4G"): [n_tile][k_block] blocks of 128 rows x 32
// bytes; each 32-bit word = 8 consecutive k as nibbles k0,k2,k4,k6,k1,k3,k5,k7
// (low to high), stored as q + 8.  Rows beyond the matrix are zero weights.
template <typename RowMap>
inline void repack_w4g(const uint8_t* packed, int64_t n_tiles, int64_t K, RowMap row_map, uint32_t* out) {
  const int64_t KB = K / 64;
  parallel_for(n_tiles, [&](int64_t nt) {
    for (int64_t kb = 0; kb < KB; ++kb) {
      uint32_t* blk = out + (nt * KB + kb) * 1024;   // 4096 bytes
      for (int r = 0; r < 128; ++r) {
        int64_t src = row_map(nt * 128 + r);
        for (int wi = 0; wi < 8; ++wi) {
          uint32_t w = 0;
          for (int e = 0; e < 8; ++e) {
            int q = src >= 0 ? canon_q(packed, K, src, kb * 64 + wi * 8 + e) : 0;
            int nib = (e & 1) ? 4 + (e >> 1) : (e >> 1);
            w |= (uint32_t)(q + 8) << (4 * nib);
          }
          blk[r * 8 + wi] = w;
        }
      }
    }
  });
}

// RoPE tables in double precision, rounded once to float (the oracle builds
// its tables with the same expressions).
inline void build_rope_table(double base, int hd, int max_ctx, std::vector<float>& cos_t, std::vector<float>& sin_t) {
  int half = hd / 2;
  cos_t.resize((size_t)max_ctx * half);
  sin_t.resize((size_t)max_ctx * half);
  for (int p = 0; p < max_ctx; ++p)
    for (int j = 0; j < half; ++j) {
      double inv = std::pow(base, -2.0 * (double)j / (double)hd);
      double a = (double)p * inv;
      cos_t[(size_t)p * half + j] = (float)std::cos(a);
      sin_t[(size_t)p * half + j] = (float)std::sin(a);
    }
}

// Prefill work groups: runtime/executor/litert_compiled_model_executor_utils.cc:300-330.
inline std::vector<std::pair<int, int>> plan_work_groups(const int* buckets, int n_buckets, int input_length) {
  std::vector<std::pair<int, int>> groups;
  int max_len = buckets[0];
  while (input_length >= max_len) {
    groups.emplace_back(max_len, max_len);
    input_length -= max_len;
  }
  if (input_length > 0) {
    for (int i = 0; i < n_buckets; ++i) {
      if (i + 1 < n_buckets && buckets[i + 1] >= input_length) continue;
      groups.emplace_back(buckets[i], input_length);
      break;
    }
  }
  return groups;
}

}  // namespace b200lm
