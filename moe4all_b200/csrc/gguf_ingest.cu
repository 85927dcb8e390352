// GGUF ingest: find the MoE FFN tensors of a model file and put their bytes on the device.
//
// The reference parses the file in crates/infr-gguf/src/lib.rs:443-1000 (single-file form:
// :745-870) and uploads expert banks byte for byte (`Rewrite::Native`,
// crates/infr-llama/src/seam/weight_upload.rs:8-14).  The same rules here: little-endian, magic
// "GGUF", versions 2 and 3, metadata key/values (arrays are skipped, scalars kept),
// `general.alignment` a power of two (default 32, capped), tensor infos (name, up to four
// dimensions with ne[0] the fastest axis, ggml type, offset relative to the aligned data region),
// a quantised tensor must be a whole number of blocks and must lie inside the file.  Malformed
// input is an error with a message, never a crash.  Split (multi-file) models are not handled.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "common.cuh"

namespace {

struct MetaScalar {
  int kind = 0;  // 1 unsigned / bool, 2 signed, 3 float
  uint64_t u = 0;
  int64_t i = 0;
  double f = 0.0;
};

struct TensorEntry {
  int32_t type = 0;
  uint32_t n_dims = 0;
  uint64_t dims[4] = {1, 1, 1, 1};
  uint64_t offset = 0;  // absolute in the file
  uint64_t nbytes = 0;  // 0: block layout of this type unknown here
};

// (elements per block, bytes per block) of the ggml types a model file may hold
bool block_layout(int32_t type, uint64_t* elems, uint64_t* bytes) {
  switch (type) {
    case 0: *elems = 1; *bytes = 4; return true;      // F32
    case 1: *elems = 1; *bytes = 2; return true;      // F16
    case 2: *elems = 32; *bytes = 18; return true;    // Q4_0
    case 3: *elems = 32; *bytes = 20; return true;    // Q4_1
    case 6: *elems = 32; *bytes = 22; return true;    // Q5_0
    case 7: *elems = 32; *bytes = 24; return true;    // Q5_1
    case 8: *elems = 32; *bytes = 34; return true;    // Q8_0
    case 10: *elems = 256; *bytes = 84; return true;  // Q2_K
    case 11: *elems = 256; *bytes = 110; return true; // Q3_K
    case 12: *elems = 256; *bytes = 144; return true; // Q4_K
    case 13: *elems = 256; *bytes = 176; return true; // Q5_K
    case 14: *elems = 256; *bytes = 210; return true; // Q6_K
    case 17: *elems = 256; *bytes = 74; return true;  // IQ2_XS
    case 18: *elems = 256; *bytes = 98; return true;  // IQ3_XXS
    case 21: *elems = 256; *bytes = 110; return true; // IQ3_S
    case 22: *elems = 256; *bytes = 82; return true;  // IQ2_S
    case 20: *elems = 32; *bytes = 18; return true;   // IQ4_NL
    case 23: *elems = 256; *bytes = 136; return true; // IQ4_XS
    case 24: *elems = 1; *bytes = 1; return true;     // I8
    case 25: *elems = 1; *bytes = 2; return true;     // I16
    case 26: *elems = 1; *bytes = 4; return true;     // I32
    case 27: *elems = 1; *bytes = 8; return true;     // I64
    case 28: *elems = 1; *bytes = 8; return true;     // F64
    case 30: *elems = 1; *bytes = 2; return true;     // BF16
    case 39: *elems = 32; *bytes = 17; return true;   // MXFP4
    case 40: *elems = 64; *bytes = 36; return true;   // NVFP4
    case 42: *elems = 64; *bytes = 18; return true;   // Q2_0
    default: return false;
  }
}

constexpr uint64_t MAX_ALIGNMENT = 1ull << 20;
constexpr int MAX_META_DEPTH = 64;

}  // namespace

struct infr_cuda_gguf {
  int fd = -1;
  const unsigned char* map = nullptr;
  size_t size = 0;
  uint32_t version = 0;
  uint64_t alignment = 32, data_start = 0;
  std::map<std::string, MetaScalar> meta;
  std::map<std::string, std::string> meta_str;
  std::map<std::string, TensorEntry> tensors;
};

namespace {

struct Reader {
  const unsigned char* p;
  size_t n, pos = 0;
  std::string err;
  bool need(size_t k) {
    if (k > n - pos) {
      char m[128];
      std::snprintf(m, sizeof m, "GGUF: unexpected end of file at offset %zu (need %zu more bytes, file is %zu bytes)", pos, k, n);
      err = m;
      return false;
    }
    return true;
  }
  template <typename T>
  bool get(T* v) {
    if (!need(sizeof(T))) return false;
    std::memcpy(v, p + pos, sizeof(T));
    pos += sizeof(T);
    return true;
  }
  bool str(std::string* s) {
    uint64_t len;
    if (!get(&len)) return false;
    if (len > n - pos) return need((size_t)-1 >> 1);
    s->assign(reinterpret_cast<const char*>(p + pos), (size_t)len);
    pos += (size_t)len;
    return true;
  }
  // one metadata value; scalars are returned, strings through `sv`, arrays skipped
  bool value(uint32_t type, MetaScalar* out, std::string* sv, int depth) {
    switch (type) {
      case 0: { uint8_t v; if (!get(&v)) return false; out->kind = 1; out->u = v; return true; }
      case 1: { int8_t v; if (!get(&v)) return false; out->kind = 2; out->i = v; return true; }
      case 2: { uint16_t v; if (!get(&v)) return false; out->kind = 1; out->u = v; return true; }
      case 3: { int16_t v; if (!get(&v)) return false; out->kind = 2; out->i = v; return true; }
      case 4: { uint32_t v; if (!get(&v)) return false; out->kind = 1; out->u = v; return true; }
      case 5: { int32_t v; if (!get(&v)) return false; out->kind = 2; out->i = v; return true; }
      case 6: { float v; if (!get(&v)) return false; out->kind = 3; out->f = v; return true; }
      case 7: { uint8_t v; if (!get(&v)) return false; out->kind = 1; out->u = v != 0; return true; }
      case 8: { out->kind = 4; return str(sv); }
      case 9: {
        if (depth >= MAX_META_DEPTH) {
          err = "GGUF: metadata array nesting exceeds the maximum depth";
          return false;
        }
        uint32_t et;
        uint64_t cnt;
        if (!get(&et) || !get(&cnt)) return false;
        for (uint64_t i = 0; i < cnt; ++i) {
          MetaScalar tmp;
          std::string ts;
          if (!value(et, &tmp, &ts, depth + 1)) return false;
        }
        out->kind = 0;
        return true;
      }
      case 10: { uint64_t v; if (!get(&v)) return false; out->kind = 1; out->u = v; return true; }
      case 11: { int64_t v; if (!get(&v)) return false; out->kind = 2; out->i = v; return true; }
      case 12: { double v; if (!get(&v)) return false; out->kind = 3; out->f = v; return true; }
      default: {
        char m[64];
        std::snprintf(m, sizeof m, "GGUF: unknown value type %u", type);
        err = m;
        return false;
      }
    }
  }
};

void put_err(char* err, size_t cap, const std::string& m) {
  if (err && cap) std::snprintf(err, cap, "%s", m.c_str());
}

bool parse(infr_cuda_gguf* g, std::string* why) {
  Reader r{g->map, g->size};
  uint32_t magic = 0;
  if (!r.get(&magic)) { *why = r.err; return false; }
  if (magic != 0x46554747u) { *why = "not a GGUF file (wrong magic)"; return false; }
  if (!r.get(&g->version)) { *why = r.err; return false; }
  if (g->version != 2 && g->version != 3) { *why = "unsupported GGUF version (supported: 2, 3)"; return false; }
  uint64_t n_tensors = 0, n_kv = 0;
  if (!r.get(&n_tensors) || !r.get(&n_kv)) { *why = r.err; return false; }
  for (uint64_t i = 0; i < n_kv; ++i) {
    std::string key, sv;
    uint32_t vt;
    MetaScalar v;
    if (!r.str(&key) || !r.get(&vt) || !r.value(vt, &v, &sv, 0)) { *why = r.err; return false; }
    if (v.kind == 4) g->meta_str[key] = sv;
    else if (v.kind) g->meta[key] = v;
  }
  auto al = g->meta.find("general.alignment");
  if (al != g->meta.end()) g->alignment = al->second.kind == 2 ? (uint64_t)al->second.i : al->second.u;
  if (g->alignment == 0 || (g->alignment & (g->alignment - 1)) || g->alignment > MAX_ALIGNMENT) {
    *why = "GGUF: invalid general.alignment (must be a power of two, at most 1 MiB)";
    return false;
  }
  struct Raw { std::string name; TensorEntry t; };
  std::vector<Raw> raw;
  for (uint64_t i = 0; i < n_tensors; ++i) {
    Raw e;
    if (!r.str(&e.name) || !r.get(&e.t.n_dims)) { *why = r.err; return false; }
    if (e.t.n_dims > 4) { *why = "GGUF: tensor '" + e.name + "' declares more than 4 dimensions"; return false; }
    for (uint32_t d = 0; d < e.t.n_dims; ++d)
      if (!r.get(&e.t.dims[d])) { *why = r.err; return false; }
    if (!r.get(&e.t.type) || !r.get(&e.t.offset)) { *why = r.err; return false; }
    raw.push_back(std::move(e));
  }
  g->data_start = (r.pos + g->alignment - 1) / g->alignment * g->alignment;
  for (Raw& e : raw) {
    unsigned __int128 numel = 1;
    for (uint32_t d = 0; d < e.t.n_dims; ++d) {
      numel *= e.t.dims[d];
      if (numel > ((unsigned __int128)1 << 62)) { *why = "GGUF: tensor '" + e.name + "' shape overflows"; return false; }
    }
    uint64_t be = 0, bb = 0;
    if (block_layout(e.t.type, &be, &bb)) {
      if ((uint64_t)numel % be) { *why = "GGUF: tensor '" + e.name + "' is not a whole number of blocks"; return false; }
      // rows are whole blocks too (llama.cpp checks ne[0] % block == 0 at load)
      if (e.t.n_dims && e.t.dims[0] % be) { *why = "GGUF: tensor '" + e.name + "' rows are not a whole number of blocks"; return false; }
      e.t.nbytes = (uint64_t)numel / be * bb;
    }
    if (e.t.offset > g->size || g->data_start > g->size - e.t.offset) { *why = "GGUF: tensor '" + e.name + "' starts beyond the end of the file"; return false; }
    e.t.offset += g->data_start;
    if (e.t.nbytes > g->size - e.t.offset) { *why = "GGUF: tensor '" + e.name + "' runs beyond the end of the file"; return false; }
    if (g->tensors.count(e.name)) { *why = "GGUF: duplicate tensor name '" + e.name + "'"; return false; }
    g->tensors[e.name] = e.t;
  }
  return true;
}

}  // namespace

extern "C" {

int32_t infr_cuda_gguf_open(const char* path, infr_cuda_gguf** out, char* err, size_t err_cap) {
  if (!path || !out) return INFR_CUDA_ERR_INVALID_ARG;
  *out = nullptr;
  infr_cuda_gguf* g = new (std::nothrow) infr_cuda_gguf();
  if (!g) return INFR_CUDA_ERR_OOM;
  g->fd = ::open(path, O_RDONLY);
  struct stat st;
  if (g->fd < 0 || ::fstat(g->fd, &st) != 0) {
    put_err(err, err_cap, std::string("GGUF: cannot open ") + path);
    infr_cuda_gguf_close(g);
    return INFR_CUDA_ERR_INVALID_ARG;
  }
  g->size = (size_t)st.st_size;
  if (g->size) {
    void* m = ::mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) {
      put_err(err, err_cap, std::string("GGUF: cannot map ") + path);
      infr_cuda_gguf_close(g);
      return INFR_CUDA_ERR_INVALID_ARG;
    }
    g->map = static_cast<const unsigned char*>(m);
  }
  std::string why;
  if (!parse(g, &why)) {
    put_err(err, err_cap, why);
    infr_cuda_gguf_close(g);
    return INFR_CUDA_ERR_INVALID_ARG;
  }
  *out = g;
  return INFR_CUDA_OK;
}

void infr_cuda_gguf_close(infr_cuda_gguf* g) {
  if (!g) return;
  if (g->map) ::munmap(const_cast<unsigned char*>(g->map), g->size);
  if (g->fd >= 0) ::close(g->fd);
  delete g;
}

uint64_t infr_cuda_gguf_tensor_count(const infr_cuda_gguf* g) { return g ? g->tensors.size() : 0; }

int32_t infr_cuda_gguf_tensor_name(const infr_cuda_gguf* g, uint64_t index, char* out, size_t cap) {
  if (!g || !out || !cap || index >= g->tensors.size()) return INFR_CUDA_ERR_INVALID_ARG;
  auto it = g->tensors.begin();
  std::advance(it, (ptrdiff_t)index);  // name order; a caller walking all names of a shard pays n^2 / 2 steps of a small map
  if (it->first.size() + 1 > cap) return INFR_CUDA_ERR_INVALID_ARG;
  std::snprintf(out, cap, "%s", it->first.c_str());
  return INFR_CUDA_OK;
}

int32_t infr_cuda_gguf_find(const infr_cuda_gguf* g, const char* name, infr_cuda_gguf_tensor* out) {
  if (!g || !name || !out) return INFR_CUDA_ERR_INVALID_ARG;
  auto it = g->tensors.find(name);
  if (it == g->tensors.end()) return INFR_CUDA_ERR_INVALID_ARG;
  out->dtype = it->second.type;
  out->n_dims = it->second.n_dims;
  for (int d = 0; d < 4; ++d) out->dims[d] = it->second.dims[d];
  out->offset = it->second.offset;
  out->nbytes = it->second.nbytes;
  return INFR_CUDA_OK;
}

int32_t infr_cuda_gguf_meta_u64(const infr_cuda_gguf* g, const char* key, uint64_t* out) {
  if (!g || !key || !out) return INFR_CUDA_ERR_INVALID_ARG;
  auto it = g->meta.find(key);
  if (it == g->meta.end() || it->second.kind == 3) return INFR_CUDA_ERR_INVALID_ARG;
  if (it->second.kind == 2 && it->second.i < 0) return INFR_CUDA_ERR_INVALID_ARG;
  *out = it->second.kind == 2 ? (uint64_t)it->second.i : it->second.u;
  return INFR_CUDA_OK;
}

int32_t infr_cuda_gguf_meta_f64(const infr_cuda_gguf* g, const char* key, double* out) {
  if (!g || !key || !out) return INFR_CUDA_ERR_INVALID_ARG;
  auto it = g->meta.find(key);
  if (it == g->meta.end()) return INFR_CUDA_ERR_INVALID_ARG;
  *out = it->second.kind == 3 ? it->second.f : it->second.kind == 2 ? (double)it->second.i : (double)it->second.u;
  return INFR_CUDA_OK;
}

int32_t infr_cuda_gguf_meta_str(const infr_cuda_gguf* g, const char* key, char* out, size_t cap) {
  if (!g || !key || !out || !cap) return INFR_CUDA_ERR_INVALID_ARG;
  auto it = g->meta_str.find(key);
  if (it == g->meta_str.end()) return INFR_CUDA_ERR_INVALID_ARG;
  std::snprintf(out, cap, "%s", it->second.c_str());
  return INFR_CUDA_OK;
}

int32_t infr_cuda_gguf_upload(infr_cuda_ctx* ctx, const infr_cuda_gguf* g, const char* name, infr_cuda_buf** out) {
  if (!ctx || !g || !name || !out) return INFR_CUDA_ERR_INVALID_ARG;
  *out = nullptr;
  auto it = g->tensors.find(name);
  if (it == g->tensors.end()) return infr::fail(ctx, INFR_CUDA_ERR_INVALID_ARG, std::string("GGUF: no tensor named '") + name + "'");
  if (!it->second.nbytes) return infr::fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, std::string("GGUF: tensor '") + name + "' has a ggml type whose block layout is not known here");
  // 16 spare bytes: the kernels' funnel-shift reads of 2-byte-aligned Q6_K blocks may touch up to
  // two bytes past the last block
  infr_cuda_buf* b = nullptr;
  int32_t rc = infr_cuda_alloc(ctx, (size_t)it->second.nbytes + 16, 1, &b);
  if (rc) return rc;
  rc = infr_cuda_upload(ctx, b, 0, g->map + it->second.offset, (size_t)it->second.nbytes);
  if (rc) {
    infr_cuda_free(ctx, b);
    return rc;
  }
  *out = b;
  return INFR_CUDA_OK;
}

}  // extern "C"
