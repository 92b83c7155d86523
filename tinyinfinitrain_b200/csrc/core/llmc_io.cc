#include "core/llmc_io.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <c10/util/Exception.h>

#include <cstdio>
#include <cstring>
#include <memory>

namespace titb {
namespace llmc {
namespace {

struct File {
  FILE* f;
  explicit File(const std::string& path, const char* mode) : f(std::fopen(path.c_str(), mode)) {
    TORCH_CHECK(f != nullptr, "File not found or not writable: ", path);
  }
  ~File() { if (f) std::fclose(f); }
  void read(void* dst, size_t n) { TORCH_CHECK(std::fread(dst, 1, n, f) == n, "unexpected end of file"); }
  void write(const void* src, size_t n) { TORCH_CHECK(std::fwrite(src, 1, n, f) == n, "short write"); }
  void skip(long n) { TORCH_CHECK(std::fseek(f, n, SEEK_CUR) == 0, "seek failed"); }
};

// Reads `numel` values stored as fp32 (version 3) or bf16 (version 5) into an fp32 tensor.
at::Tensor read_block(File& in, std::vector<int64_t> shape, int32_t version) {
  at::Tensor t = at::empty(shape, at::kFloat);
  const int64_t n = t.numel();
  if (version == kVersionFp32) {
    in.read(t.data_ptr<float>(), sizeof(float) * n);
  } else {
    at::Tensor raw = at::empty(shape, at::kBFloat16);
    in.read(raw.data_ptr(), 2 * n);
    t.copy_(raw);
  }
  return t;
}
void write_block(File& out, const at::Tensor& t, int32_t version) {
  if (version == kVersionFp32) {
    at::Tensor c = t.detach().to(at::kCPU, at::kFloat).contiguous();
    out.write(c.data_ptr<float>(), sizeof(float) * c.numel());
  } else {
    at::Tensor c = t.detach().to(at::kCPU, at::kBFloat16).contiguous();
    out.write(c.data_ptr(), 2 * c.numel());
  }
}
const at::Tensor& get(const StateDict& sd, const std::string& k) {
  auto it = sd.find(k);
  TORCH_CHECK(it != sd.end(), "state dict has no entry ", k);
  return it->second;
}
std::string layer_key(int l, const char* suffix) { return "transformer.h." + std::to_string(l) + "." + suffix; }

struct Kind { const char* name; int64_t rows, cols; };  // cols == 0: vector of `rows`

}  // namespace

Gpt2Header read_gpt2_header(const std::string& path) {
  File in(path, "rb");
  int32_t h[256];
  in.read(h, sizeof(h));
  TORCH_CHECK(h[0] == kGpt2Magic, "not an llm.c GPT-2 checkpoint (magic ", h[0], ")");
  TORCH_CHECK(h[1] == kVersionFp32 || h[1] == kVersionBf16, "unsupported checkpoint version ", h[1]);
  Gpt2Header r;
  r.version = h[1]; r.block_size = h[2]; r.vocab_size = h[3]; r.n_layer = h[4]; r.n_head = h[5]; r.n_embd = h[6];
  r.padded_vocab_size = h[7];
  return r;
}

static std::vector<Kind> gpt2_kinds(int64_t C) {
  return {{"ln_1.weight", C, 0}, {"ln_1.bias", C, 0}, {"attn.c_attn.weight", 3 * C, C}, {"attn.c_attn.bias", 3 * C, 0},
          {"attn.c_proj.weight", C, C}, {"attn.c_proj.bias", C, 0}, {"ln_2.weight", C, 0}, {"ln_2.bias", C, 0},
          {"mlp.c_fc.weight", 4 * C, C}, {"mlp.c_fc.bias", 4 * C, 0}, {"mlp.c_proj.weight", C, 4 * C},
          {"mlp.c_proj.bias", C, 0}};
}

StateDict read_gpt2(const std::string& path, Gpt2Header* header_out, bool keep_padding) {
  const Gpt2Header h = read_gpt2_header(path);
  if (header_out) *header_out = h;
  File in(path, "rb");
  in.skip(256 * sizeof(int32_t));
  const int64_t C = h.n_embd, L = h.n_layer;
  const long esz = h.version == kVersionFp32 ? 4 : 2;
  StateDict sd;
  const int64_t keep = keep_padding ? h.padded_vocab_size : h.vocab_size;
  sd["transformer.wte.weight"] = read_block(in, {keep, C}, h.version);
  in.skip((h.padded_vocab_size - keep) * C * esz);
  sd["transformer.wpe.weight"] = read_block(in, {h.block_size, C}, h.version);
  for (const Kind& k : gpt2_kinds(C))
    for (int l = 0; l < L; ++l)
      sd[layer_key(l, k.name)] = k.cols ? read_block(in, {k.rows, k.cols}, h.version) : read_block(in, {k.rows}, h.version);
  sd["transformer.ln_f.weight"] = read_block(in, {C}, h.version);
  sd["transformer.ln_f.bias"] = read_block(in, {C}, h.version);
  sd["lm_head.weight"] = sd["transformer.wte.weight"];  // tied
  return sd;
}

void write_gpt2(const std::string& path, const Gpt2Header& h, const StateDict& sd) {
  File out(path, "wb");
  int32_t hdr[256];
  std::memset(hdr, 0, sizeof(hdr));
  hdr[0] = kGpt2Magic; hdr[1] = h.version; hdr[2] = h.block_size; hdr[3] = h.vocab_size; hdr[4] = h.n_layer;
  hdr[5] = h.n_head; hdr[6] = h.n_embd; hdr[7] = h.padded_vocab_size;
  out.write(hdr, sizeof(hdr));
  const int64_t C = h.n_embd;
  at::Tensor wte = get(sd, "transformer.wte.weight").detach().to(at::kCPU, at::kFloat);
  TORCH_CHECK(wte.size(0) >= h.vocab_size && wte.size(1) == C, "wte has the wrong shape");
  at::Tensor padded = at::zeros({h.padded_vocab_size, C}, at::kFloat);
  const int64_t rows = std::min<int64_t>(wte.size(0), h.padded_vocab_size);
  padded.narrow(0, 0, rows).copy_(wte.narrow(0, 0, rows));
  write_block(out, padded, h.version);
  write_block(out, get(sd, "transformer.wpe.weight"), h.version);
  for (const Kind& k : gpt2_kinds(C))
    for (int l = 0; l < h.n_layer; ++l) write_block(out, get(sd, layer_key(l, k.name)), h.version);
  write_block(out, get(sd, "transformer.ln_f.weight"), h.version);
  write_block(out, get(sd, "transformer.ln_f.bias"), h.version);
}

// ---------------------------------------------------------------------------- LLaMA-3
static std::vector<Kind> llama3_kinds(const Llama3Header& h) {
  const int64_t C = h.n_embd, hd = C / h.n_head, F = h.ffn_dim;
  return {{"ln_1.weight", C, 0}, {"attn.c_attn.weight", (h.n_head + 2 * h.n_kv_head) * hd, C},
          {"attn.c_proj.weight", C, C}, {"ln_2.weight", C, 0}, {"mlp.c_fc.weight", 2 * F, C},
          {"mlp.c_proj.weight", C, F}};
}

Llama3Header read_llama3_header(const std::string& path) {
  File in(path, "rb");
  int32_t h[256];
  in.read(h, sizeof(h));
  TORCH_CHECK(h[0] == kLlama3Magic, "not a LLaMA-3 checkpoint of this framework (magic ", h[0], ")");
  TORCH_CHECK(h[1] == kVersionFp32 || h[1] == kVersionBf16, "unsupported checkpoint version ", h[1]);
  Llama3Header r;
  r.version = h[1]; r.max_seq_len = h[2]; r.vocab_size = h[3]; r.n_layer = h[4]; r.n_head = h[5]; r.n_kv_head = h[6];
  r.n_embd = h[7]; r.ffn_dim = h[8];
  std::memcpy(&r.rope_theta, &h[9], 4);
  std::memcpy(&r.norm_eps, &h[10], 4);
  return r;
}

StateDict read_llama3(const std::string& path, Llama3Header* header_out) {
  const Llama3Header h = read_llama3_header(path);
  if (header_out) *header_out = h;
  File in(path, "rb");
  in.skip(256 * sizeof(int32_t));
  StateDict sd;
  sd["transformer.wte.weight"] = read_block(in, {h.vocab_size, h.n_embd}, h.version);
  for (const Kind& k : llama3_kinds(h))
    for (int l = 0; l < h.n_layer; ++l)
      sd[layer_key(l, k.name)] = k.cols ? read_block(in, {k.rows, k.cols}, h.version) : read_block(in, {k.rows}, h.version);
  sd["transformer.ln_f.weight"] = read_block(in, {h.n_embd}, h.version);
  sd["lm_head.weight"] = read_block(in, {h.vocab_size, h.n_embd}, h.version);
  return sd;
}

void write_llama3(const std::string& path, const Llama3Header& h, const StateDict& sd) {
  File out(path, "wb");
  int32_t hdr[256];
  std::memset(hdr, 0, sizeof(hdr));
  hdr[0] = kLlama3Magic; hdr[1] = h.version; hdr[2] = h.max_seq_len; hdr[3] = h.vocab_size; hdr[4] = h.n_layer;
  hdr[5] = h.n_head; hdr[6] = h.n_kv_head; hdr[7] = h.n_embd; hdr[8] = h.ffn_dim;
  std::memcpy(&hdr[9], &h.rope_theta, 4);
  std::memcpy(&hdr[10], &h.norm_eps, 4);
  out.write(hdr, sizeof(hdr));
  write_block(out, get(sd, "transformer.wte.weight").narrow(0, 0, h.vocab_size), h.version);
  for (const Kind& k : llama3_kinds(h))
    for (int l = 0; l < h.n_layer; ++l) write_block(out, get(sd, layer_key(l, k.name)), h.version);
  write_block(out, get(sd, "transformer.ln_f.weight"), h.version);
  write_block(out, get(sd, "lm_head.weight").narrow(0, 0, h.vocab_size), h.version);
}


// ---------------------------------------------------------------------------- memory-mapped views
namespace {
struct Mapping {
  void* base = MAP_FAILED;
  size_t bytes = 0;
  ~Mapping() { if (base != MAP_FAILED) munmap(base, bytes); }
};
std::shared_ptr<Mapping> map_file(const std::string& path) {
  const int fd = open(path.c_str(), O_RDONLY | O_CLOEXEC);
  TORCH_CHECK(fd >= 0, "cannot open ", path);
  struct stat st;
  if (fstat(fd, &st) != 0) { close(fd); TORCH_CHECK(false, "cannot stat ", path); }
  auto m = std::make_shared<Mapping>();
  m->bytes = static_cast<size_t>(st.st_size);
  m->base = mmap(nullptr, m->bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE, fd, 0);
  close(fd);
  TORCH_CHECK(m->base != MAP_FAILED, "cannot map ", path);
  return m;
}
// Hands out consecutive blocks of the payload as tensors that keep the mapping alive.
struct BlockCursor {
  std::shared_ptr<Mapping> map;
  size_t pos;
  int version;
  at::Tensor next(std::vector<int64_t> shape) {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    const size_t esz = version == kVersionFp32 ? 4 : 2;
    TORCH_CHECK(pos + n * esz <= map->bytes, "checkpoint file is shorter than its header implies");
    auto keep = map;
    at::Tensor t = at::from_blob(static_cast<char*>(map->base) + pos, shape, [keep](void*) mutable { keep.reset(); },
                                 at::TensorOptions().dtype(version == kVersionFp32 ? at::kFloat : at::kBFloat16));
    pos += n * esz;
    return t;
  }
};
}  // namespace

StateDict map_gpt2(const std::string& path, Gpt2Header* header_out) {
  const Gpt2Header h = read_gpt2_header(path);
  if (header_out) *header_out = h;
  BlockCursor cur{map_file(path), 256 * sizeof(int32_t), h.version};
  const int64_t C = h.n_embd;
  StateDict sd;
  sd["transformer.wte.weight"] = cur.next({h.padded_vocab_size, C});
  sd["transformer.wpe.weight"] = cur.next({h.block_size, C});
  for (const Kind& k : gpt2_kinds(C))
    for (int l = 0; l < h.n_layer; ++l)
      sd[layer_key(l, k.name)] = k.cols ? cur.next({k.rows, k.cols}) : cur.next({k.rows});
  sd["transformer.ln_f.weight"] = cur.next({C});
  sd["transformer.ln_f.bias"] = cur.next({C});
  sd["lm_head.weight"] = sd["transformer.wte.weight"];  // tied
  return sd;
}

StateDict map_llama3(const std::string& path, Llama3Header* header_out) {
  const Llama3Header h = read_llama3_header(path);
  if (header_out) *header_out = h;
  BlockCursor cur{map_file(path), 256 * sizeof(int32_t), h.version};
  StateDict sd;
  sd["transformer.wte.weight"] = cur.next({h.vocab_size, h.n_embd});
  for (const Kind& k : llama3_kinds(h))
    for (int l = 0; l < h.n_layer; ++l)
      sd[layer_key(l, k.name)] = k.cols ? cur.next({k.rows, k.cols}) : cur.next({k.rows});
  sd["transformer.ln_f.weight"] = cur.next({h.n_embd});
  sd["lm_head.weight"] = cur.next({h.vocab_size, h.n_embd});
  return sd;
}

// ----------------------------------------------------------------------------- tokens
at::Tensor read_tokens(const std::string& path, int32_t* magic_out) {
  File in(path, "rb");
  int32_t h[256];
  in.read(h, sizeof(h));
  TORCH_CHECK(h[0] == kDataMagicU16 || h[0] == kDataMagicU32, "unknown token file magic ", h[0]);
  if (magic_out) *magic_out = h[0];
  const int64_t n = static_cast<uint32_t>(h[2]);
  at::Tensor out = at::empty({n}, at::kLong);
  int64_t* dst = out.data_ptr<int64_t>();
  if (h[0] == kDataMagicU16) {
    std::vector<uint16_t> buf(n);
    in.read(buf.data(), 2 * n);
    for (int64_t i = 0; i < n; ++i) dst[i] = buf[i];
  } else {
    std::vector<uint32_t> buf(n);
    in.read(buf.data(), 4 * n);
    for (int64_t i = 0; i < n; ++i) dst[i] = buf[i];
  }
  return out;
}

void write_tokens(const std::string& path, const at::Tensor& tokens, int32_t magic) {
  TORCH_CHECK(magic == kDataMagicU16 || magic == kDataMagicU32, "unknown token file magic ", magic);
  at::Tensor t = tokens.to(at::kCPU, at::kLong).contiguous();
  File out(path, "wb");
  int32_t hdr[256];
  std::memset(hdr, 0, sizeof(hdr));
  hdr[0] = magic; hdr[1] = magic == kDataMagicU16 ? 1 : 7; hdr[2] = static_cast<int32_t>(t.numel());
  out.write(hdr, sizeof(hdr));
  const int64_t* src = t.data_ptr<int64_t>();
  if (magic == kDataMagicU16) {
    std::vector<uint16_t> buf(t.numel());
    for (int64_t i = 0; i < t.numel(); ++i) buf[i] = static_cast<uint16_t>(src[i]);
    out.write(buf.data(), 2 * buf.size());
  } else {
    std::vector<uint32_t> buf(t.numel());
    for (int64_t i = 0; i < t.numel(); ++i) buf[i] = static_cast<uint32_t>(src[i]);
    out.write(buf.data(), 4 * buf.size());
  }
}

}  // namespace llmc
}  // namespace titb
