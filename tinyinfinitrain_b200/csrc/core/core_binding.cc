// Python bindings of the C++ framework core: RNG, llm.c file formats, datasets, tokenizer.
#include <torch/extension.h>

#include "core/data.h"
#include "core/llmc_io.h"
#include "core/rng.h"

namespace {

std::optional<uint32_t> opt_seed(const c10::optional<int64_t>& s) {
  if (s.has_value()) return static_cast<uint32_t>(*s);
  return std::nullopt;
}

void rng_normal_(at::Tensor t, double mean, double std, c10::optional<int64_t> seed) {
  TORCH_CHECK(t.device().is_cpu() && t.scalar_type() == at::kFloat && t.is_contiguous(),
              "rng_normal_: contiguous CPU float tensor expected");
  titb::rng::fill_normal(t.data_ptr<float>(), t.numel(), (float)mean, (float)std, opt_seed(seed));
}
void rng_uniform_(at::Tensor t, double lo, double hi, c10::optional<int64_t> seed) {
  TORCH_CHECK(t.device().is_cpu() && t.scalar_type() == at::kFloat && t.is_contiguous(),
              "rng_uniform_: contiguous CPU float tensor expected");
  titb::rng::fill_uniform(t.data_ptr<float>(), t.numel(), (float)lo, (float)hi, opt_seed(seed));
}
void rng_randint_(at::Tensor t, int64_t lo, int64_t hi, int64_t seed) {
  TORCH_CHECK(t.device().is_cpu() && t.scalar_type() == at::kLong && t.is_contiguous(),
              "rng_randint_: contiguous CPU int64 tensor expected");
  titb::rng::fill_randint(t.data_ptr<int64_t>(), t.numel(), lo, hi, (uint32_t)seed);
}

py::dict gpt2_header_dict(const titb::llmc::Gpt2Header& h) {
  py::dict d;
  d["version"] = h.version; d["block_size"] = h.block_size; d["vocab_size"] = h.vocab_size;
  d["n_layer"] = h.n_layer; d["n_head"] = h.n_head; d["n_embd"] = h.n_embd;
  d["padded_vocab_size"] = h.padded_vocab_size;
  return d;
}
titb::llmc::Gpt2Header gpt2_header_from(const py::dict& d) {
  titb::llmc::Gpt2Header h;
  h.version = d["version"].cast<int>(); h.block_size = d["block_size"].cast<int>();
  h.vocab_size = d["vocab_size"].cast<int>(); h.n_layer = d["n_layer"].cast<int>();
  h.n_head = d["n_head"].cast<int>(); h.n_embd = d["n_embd"].cast<int>();
  h.padded_vocab_size = d["padded_vocab_size"].cast<int>();
  return h;
}
py::dict llama3_header_dict(const titb::llmc::Llama3Header& h) {
  py::dict d;
  d["version"] = h.version; d["max_seq_len"] = h.max_seq_len; d["vocab_size"] = h.vocab_size;
  d["n_layer"] = h.n_layer; d["n_head"] = h.n_head; d["n_kv_head"] = h.n_kv_head; d["n_embd"] = h.n_embd;
  d["ffn_dim"] = h.ffn_dim; d["rope_theta"] = h.rope_theta; d["norm_eps"] = h.norm_eps;
  return d;
}
titb::llmc::Llama3Header llama3_header_from(const py::dict& d) {
  titb::llmc::Llama3Header h;
  h.version = d["version"].cast<int>(); h.max_seq_len = d["max_seq_len"].cast<int>();
  h.vocab_size = d["vocab_size"].cast<int>(); h.n_layer = d["n_layer"].cast<int>();
  h.n_head = d["n_head"].cast<int>(); h.n_kv_head = d["n_kv_head"].cast<int>();
  h.n_embd = d["n_embd"].cast<int>(); h.ffn_dim = d["ffn_dim"].cast<int>();
  h.rope_theta = d["rope_theta"].cast<float>(); h.norm_eps = d["norm_eps"].cast<float>();
  return h;
}

}  // namespace

void bind_framework(pybind11::module_& m);

void bind_core(pybind11::module_& m) {
  namespace td = titb::data;
  m.def("rng_seed", [](int64_t s) { titb::rng::seed_global((uint32_t)s); });
  m.def("rng_normal_", &rng_normal_, py::arg("t"), py::arg("mean"), py::arg("std"), py::arg("seed") = py::none());
  m.def("rng_uniform_", &rng_uniform_, py::arg("t"), py::arg("lo"), py::arg("hi"), py::arg("seed") = py::none());
  m.def("rng_randint_", &rng_randint_);

  m.def("llmc_read_gpt2", [](const std::string& path, bool keep_padding) {
    titb::llmc::Gpt2Header h;
    auto sd = titb::llmc::read_gpt2(path, &h, keep_padding);
    return py::make_tuple(gpt2_header_dict(h), sd);
  }, py::arg("path"), py::arg("keep_padding") = false);
  m.def("llmc_map_gpt2", [](const std::string& path) {
    titb::llmc::Gpt2Header h;
    auto sd = titb::llmc::map_gpt2(path, &h);
    return py::make_tuple(gpt2_header_dict(h), sd);
  });
  m.def("llmc_map_llama3", [](const std::string& path) {
    titb::llmc::Llama3Header h;
    auto sd = titb::llmc::map_llama3(path, &h);
    return py::make_tuple(llama3_header_dict(h), sd);
  });
  m.def("llmc_write_gpt2", [](const std::string& path, const py::dict& header, const titb::llmc::StateDict& sd) {
    titb::llmc::write_gpt2(path, gpt2_header_from(header), sd);
  });
  m.def("llmc_read_llama3", [](const std::string& path) {
    titb::llmc::Llama3Header h;
    auto sd = titb::llmc::read_llama3(path, &h);
    return py::make_tuple(llama3_header_dict(h), sd);
  });
  m.def("llmc_write_llama3", [](const std::string& path, const py::dict& header, const titb::llmc::StateDict& sd) {
    titb::llmc::write_llama3(path, llama3_header_from(header), sd);
  });
  m.def("llmc_read_tokens", [](const std::string& path) {
    int32_t magic = 0;
    at::Tensor t = titb::llmc::read_tokens(path, &magic);
    return py::make_tuple(t, magic);
  });
  m.def("llmc_write_tokens", &titb::llmc::write_tokens);

  py::class_<td::Dataset, std::shared_ptr<td::Dataset>>(m, "Dataset")
      .def("Size", &td::Dataset::Size)
      .def("__len__", &td::Dataset::Size)
      .def("SequenceLength", &td::Dataset::SequenceLength)
      .def("__getitem__", [](const td::Dataset& d, size_t i) {
        if (i >= d.Size()) throw py::index_error();
        return d.Get(i);
      });
  py::class_<td::TinyShakespeareDataset, td::Dataset, std::shared_ptr<td::TinyShakespeareDataset>>(
      m, "TinyShakespeareDataset")
      .def(py::init<const std::string&, size_t>(), py::arg("filepath"), py::arg("sequence_length"))
      .def("NumTokens", &td::TinyShakespeareDataset::NumTokens)
      .def("is_uint32", [](const td::TinyShakespeareDataset& d) {
        return d.type() == td::TinyShakespeareDataset::TinyShakespeareType::kUINT32;
      });
  py::class_<td::SyntheticDataset, td::Dataset, std::shared_ptr<td::SyntheticDataset>>(m, "SyntheticDataset")
      .def(py::init<uint32_t, int64_t, size_t, size_t>(), py::arg("seed"), py::arg("vocab_size"),
           py::arg("sequence_length"), py::arg("num_samples"));
  py::class_<td::DataLoader>(m, "DataLoader")
      .def(py::init<std::shared_ptr<td::Dataset>, size_t, bool, size_t, size_t, bool>(), py::arg("dataset"),
           py::arg("batch_size"), py::arg("pin_memory") = false, py::arg("rank") = 0, py::arg("world") = 1,
           py::arg("drop_last") = false)
      .def("NumBatches", &td::DataLoader::NumBatches)
      .def("__len__", &td::DataLoader::NumBatches)
      .def("Batch", &td::DataLoader::Batch)
      .def("__getitem__", [](const td::DataLoader& d, size_t i) {
        if (i >= d.NumBatches()) throw py::index_error();
        return d.Batch(i);
      });
  py::class_<td::Tokenizer>(m, "Tokenizer")
      .def(py::init<const std::string&>())
      .def("Decode", [](const td::Tokenizer& t, uint32_t id) { return py::bytes(t.Decode(id)); })
      .def("GetEndToken", &td::Tokenizer::GetEndToken)
      .def("VocabSize", &td::Tokenizer::VocabSize)
      .def("Magic", &td::Tokenizer::Magic)
      .def("Prompt", &td::Tokenizer::Prompt);
  m.def("write_tokenizer", &td::WriteTokenizer);
  m.def("random_u32", [](uint64_t state) { uint32_t r = td::RandomU32(&state); return py::make_tuple(r, state); });
  m.def("random_f32", [](uint64_t state) { float r = td::RandomF32(&state); return py::make_tuple(r, state); });
  m.def("sample_mult", [](const at::Tensor& probs, double coin) {
    at::Tensor p = probs.to(at::kCPU, at::kFloat).contiguous();
    return td::SampleMult(p.data_ptr<float>(), (int)p.numel(), (float)coin);
  });
  bind_framework(m);
}
