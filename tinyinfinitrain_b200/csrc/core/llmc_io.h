// llm.c binary formats: GPT-2 / LLaMA-3 checkpoints, token datasets, tokenizer tables.
//
// GPT-2 checkpoint (example/gpt2/net.cc:242-374 reads version 3; this reader/writer also
// handles version 5, the bf16 payload of gpt2_124M_bf16.bin):
//   header  256 x int32: [0] magic 20240326, [1] version (3 = fp32, 5 = bf16), [2] block_size,
//           [3] vocab_size, [4] n_layer, [5] n_head, [6] n_embd, [7] padded_vocab_size
//   payload wte[padded_vocab, C], wpe[block, C], then per kind over all layers:
//           ln_1.w, ln_1.b, c_attn.w, c_attn.b, attn.c_proj.w, attn.c_proj.b, ln_2.w, ln_2.b,
//           c_fc.w, c_fc.b, mlp.c_proj.w, mlp.c_proj.b, then ln_f.w, ln_f.b.
// LLaMA-3 checkpoint (the layout of llm.c's train_llama3.py export; the reference tree only
// carries the dataset magic 20240801): header 256 x int32: [0] magic 20240803, [1] version
// (3 = fp32, 5 = bf16), [2] max_seq_len, [3] vocab_size, [4] n_layer, [5] n_head, [6] n_kv_head,
// [7] n_embd, [8] ffn_dim, [9] rope_theta (float bits), [10] norm_eps (float bits); payload
// wte, per kind over layers: ln_1.w, c_attn.w (q|k|v rows), attn.c_proj.w, ln_2.w,
// c_fc.w (gate|up rows), mlp.c_proj.w, then ln_f.w, lm_head.w.
#pragma once
#include <ATen/ATen.h>

#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace titb {
namespace llmc {

constexpr int32_t kGpt2Magic = 20240326;
constexpr int32_t kLlama3Magic = 20240803;
constexpr int32_t kVersionFp32 = 3;
constexpr int32_t kVersionBf16 = 5;

struct Gpt2Header {
  int32_t version = kVersionFp32;
  int32_t block_size = 0, vocab_size = 0, n_layer = 0, n_head = 0, n_embd = 0, padded_vocab_size = 0;
};
struct Llama3Header {
  int32_t version = kVersionFp32;
  int32_t max_seq_len = 0, vocab_size = 0, n_layer = 0, n_head = 0, n_kv_head = 0, n_embd = 0, ffn_dim = 0;
  float rope_theta = 500000.f, norm_eps = 1e-5f;
};

using StateDict = std::map<std::string, at::Tensor>;

// Tensors come back as fp32 CPU tensors keyed by the module's StateDict names; wte keeps
// `rows_wte` rows (pass padded_vocab_size to keep the padding rows, vocab_size to drop them).
Gpt2Header read_gpt2_header(const std::string& path);
StateDict read_gpt2(const std::string& path, Gpt2Header* header_out, bool keep_padding);
void write_gpt2(const std::string& path, const Gpt2Header& header, const StateDict& sd);

// Memory-mapped views of the same tensors (no copy, pages are read when touched): fp32 payloads map to float
// tensors, bf16 payloads to bfloat16 tensors; GPT-2's wte keeps all padded rows.  A tensor-parallel rank slices
// its rows / columns out of these views, so it only ever reads its own part of a large file.  The mapping is
// private (copy-on-write) and lives as long as any returned tensor.
StateDict map_gpt2(const std::string& path, Gpt2Header* header_out);
StateDict map_llama3(const std::string& path, Llama3Header* header_out);

Llama3Header read_llama3_header(const std::string& path);
StateDict read_llama3(const std::string& path, Llama3Header* header_out);
void write_llama3(const std::string& path, const Llama3Header& header, const StateDict& sd);

// Token dataset .bin: 1024-byte header {magic, version, num_tokens}; magic 20240520 -> uint16
// tokens (GPT-2), 20240801 -> uint32 tokens (LLaMA-3).  Returned widened to int64.
constexpr int32_t kDataMagicU16 = 20240520;
constexpr int32_t kDataMagicU32 = 20240801;
at::Tensor read_tokens(const std::string& path, int32_t* magic_out);
void write_tokens(const std::string& path, const at::Tensor& tokens_i64, int32_t magic);

}  // namespace llmc
}  // namespace titb
