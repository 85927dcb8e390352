// Drives one MoE FFN layer through the C++ host mirror (include/infr_cuda.hpp) the way the
// reference's op loop drives a backend: model-owned buffers, upload, one Op::MoeFfn, download;
// then the same op compiled into a plan and executed.  Also checks the error behaviour the trait
// promises (crates/infr-core/src/backend.rs:22-33): caller mistakes come back as errors.
//
//   host_mirror_check <layer.bin> <out.bin>
// layer.bin: int32 {rows, ne, n_expert, n_used, n_ff, sh_ff, gated, 0}, then router f32, gate, up,
// down, [sh_gate, sh_up, sh_down, sh_gate_inp f32] bytes, x f32.   out.bin: dst f32, ids i32, wts f32.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "infr_cuda.hpp"

using namespace infr_cuda;

static std::vector<unsigned char> take(FILE* f, size_t n) {
  std::vector<unsigned char> v(n);
  if (n && std::fread(v.data(), 1, n, f) != n) {
    std::fprintf(stderr, "short read\n");
    std::exit(2);
  }
  return v;
}

#define CHECK(cond, what)                                   \
  do {                                                      \
    if (!(cond)) {                                          \
      std::fprintf(stderr, "check failed: %s\n", what);     \
      return 1;                                             \
    }                                                       \
  } while (0)
#define OK(status_expr)                                                                  \
  do {                                                                                   \
    Status s_ = (status_expr);                                                           \
    if (!s_.ok()) {                                                                      \
      std::fprintf(stderr, "%s: %s (%d)\n", #status_expr, s_.message.c_str(), s_.code);  \
      return 1;                                                                          \
    }                                                                                    \
  } while (0)

int main(int argc, char** argv) {
  if (argc != 3) return 2;
  FILE* f = std::fopen(argv[1], "rb");
  if (!f) return 2;
  int32_t hdr[8];
  if (std::fread(hdr, 4, 8, f) != 8) return 2;
  const uint32_t rows = hdr[0], ne = hdr[1], E = hdr[2], k = hdr[3], nff = hdr[4], sh_ff = hdr[5];
  const bool gated = hdr[6] != 0;
  const size_t q4row = ne / 256 * 144, q6row = nff / 256 * 210, q6row_sh = sh_ff ? sh_ff / 256 * 210 : 0;
  auto router = take(f, (size_t)E * ne * 4), gate = take(f, (size_t)E * nff * q4row), up = take(f, (size_t)E * nff * q4row),
       down = take(f, (size_t)E * ne * q6row);
  std::vector<unsigned char> shg, shu, shd, shi;
  if (sh_ff) {
    shg = take(f, (size_t)sh_ff * q4row);
    shu = take(f, (size_t)sh_ff * q4row);
    shd = take(f, (size_t)ne * q6row_sh);
    if (gated) shi = take(f, (size_t)ne * 4);
  }
  auto x = take(f, (size_t)rows * ne * 4);
  std::fclose(f);

  Result<Backend> made = Backend::create(0);
  CHECK(made.ok(), "Backend::create");
  Backend be = std::move(made.value);
  CHECK(be.name() == "cuda-sm100a", "name");
  CHECK(!be.capabilities().unified_memory && be.capabilities().graph_input_inplace, "capabilities");

  // alloc is zero-initialised (the calloc contract)
  {
    Result<Buffer> z = be.alloc(4096);
    CHECK(z.ok() && z.value.len_bytes() == 4096, "alloc");
    std::vector<unsigned char> back(4096, 0xAB);
    OK(be.download(z.value, back.data(), back.size()));
    for (unsigned char c : back) CHECK(c == 0, "alloc returns zeroed memory");
    // a copy beyond the buffer is an error value, and the backend stays usable
    Status s = be.upload(z.value, back.data(), 4096, 16);
    CHECK(!s.ok() && s.kind == ErrorKind::Backend && s.code == INFR_CUDA_ERR_INVALID_ARG && !s.message.empty(), "out-of-range upload is an error");
  }

  auto b_router = be.from_host(router), b_gate = be.from_host(gate), b_up = be.from_host(up), b_down = be.from_host(down), b_x = be.from_host(x);
  CHECK(b_router.ok() && b_gate.ok() && b_up.ok() && b_down.ok() && b_x.ok(), "weight upload");
  Result<Buffer> b_shg, b_shu, b_shd, b_shi;
  if (sh_ff) {
    b_shg = be.from_host(shg);
    b_shu = be.from_host(shu);
    b_shd = be.from_host(shd);
    CHECK(b_shg.ok() && b_shu.ok() && b_shd.ok(), "shared expert upload");
    if (gated) {
      b_shi = be.from_host(shi);
      CHECK(b_shi.ok(), "gate vector upload");
    }
  }
  auto b_dst = be.alloc((size_t)rows * ne * 4), b_ids = be.alloc((size_t)rows * k * 4), b_wts = be.alloc((size_t)rows * k * 4);
  CHECK(b_dst.ok() && b_ids.ok() && b_wts.ok(), "output alloc");

  MoeFfn op;
  op.x = &b_x.value;
  op.router = &b_router.value;
  op.gate_exps = &b_gate.value;
  op.up_exps = &b_up.value;
  op.down_exps = &b_down.value;
  op.dst = &b_dst.value;
  op.ids_out = &b_ids.value;
  op.wts_out = &b_wts.value;
  op.rows = rows;
  op.ne = ne;
  op.n_expert = E;
  op.n_used = k;
  op.n_ff_exp = nff;
  if (sh_ff) {
    op.sh_gate = &b_shg.value;
    op.sh_up = &b_shu.value;
    op.sh_down = &b_shd.value;
    op.sh_gate_inp = gated ? &b_shi.value : nullptr;
    op.sh_ff = sh_ff;
  }

  // a dtype without a kernel is Error::Unsupported, not a fallback
  {
    MoeFfn bad = op;
    bad.router_dtype = DType::Q4K;
    Status s = be.moe_ffn(bad);
    CHECK(!s.ok() && s.kind == ErrorKind::Unsupported, "unsupported router dtype");
  }

  OK(be.moe_ffn(op));
  OK(be.sync());
  std::vector<float> dst((size_t)rows * ne), wts((size_t)rows * k);
  std::vector<int32_t> ids((size_t)rows * k);
  OK(be.download(b_dst.value, dst.data(), dst.size() * 4));
  OK(be.download(b_ids.value, ids.data(), ids.size() * 4));
  OK(be.download(b_wts.value, wts.data(), wts.size() * 4));

  // compile once, execute: same bytes as the eager call
  OK(be.begin_record());
  OK(be.moe_ffn(op));
  Result<Plan> plan = be.end_record();
  CHECK(plan.ok() && plan.value.valid(), "end_record");
  std::vector<float> zero(dst.size(), 0.f), again(dst.size());
  OK(be.upload(b_dst.value, zero.data(), zero.size() * 4));
  OK(be.execute(plan.value));
  OK(be.sync());
  OK(be.download(b_dst.value, again.data(), again.size() * 4));
  CHECK(std::memcmp(again.data(), dst.data(), dst.size() * 4) == 0, "plan replay equals the eager result");

  FILE* o = std::fopen(argv[2], "wb");
  if (!o) return 2;
  std::fwrite(dst.data(), 4, dst.size(), o);
  std::fwrite(ids.data(), 4, ids.size(), o);
  std::fwrite(wts.data(), 4, wts.size(), o);
  std::fclose(o);
  std::puts("OK");
  return 0;
}
