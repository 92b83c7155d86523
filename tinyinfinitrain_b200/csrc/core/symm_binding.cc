// Python binding of the symmetric-memory heap (core/symm_heap.h).
#include <torch/extension.h>

#include "core/symm_heap.h"

namespace py = pybind11;
using titb::symm::Heap;

namespace {

py::dict to_dict(const titb::symm::Allocation& a) {
  py::dict d;
  d["bytes"] = a.bytes;
  d["ptrs"] = a.ptrs;
  d["mc_ptr"] = a.mc_ptr;
  return d;
}

struct PyHeap {
  std::unique_ptr<Heap> heap;
  bool host = false;
  int device = 0;
};

}  // namespace

void bind_symm(py::module_& m) {
  py::class_<PyHeap>(m, "SymmHeap")
      .def(py::init([](int rank, int world, int device, const std::string& key, const std::string& driver, bool multicast) {
             auto h = std::make_unique<PyHeap>();
             h->host = driver == "host";
             h->device = device;
             titb::symm::DriverApi api;
             if (h->host) {
               api = titb::symm::host_memory_driver();
             } else {
               TORCH_CHECK(driver == "cuda", "SymmHeap: driver must be 'cuda' or 'host'");
               auto l = titb::symm::load_cuda_driver();
               TORCH_CHECK(l.ok, "SymmHeap: ", l.error);
               api = l.api;
             }
             h->heap = std::make_unique<Heap>(rank, world, device, key, api, multicast);
             return h;
           }),
           py::arg("rank"), py::arg("world"), py::arg("device"), py::arg("key"), py::arg("driver") = "cuda",
           py::arg("multicast") = true)
      .def("set_timeout", [](PyHeap& h, double s) { h.heap->socket_timeout_s = s; })
      .def("listen", [](PyHeap& h) { h.heap->listen(); })
      .def("exchange", [](PyHeap& h, size_t bytes) { return h.heap->exchange(bytes); },
           py::call_guard<py::gil_scoped_release>())
      .def("multicast_ready", [](PyHeap& h, int id) { return h.heap->multicast_ready(id); })
      .def("finish", [](PyHeap& h, int id, bool use_mc) { return to_dict(h.heap->finish(id, use_mc)); }, py::arg("id"),
           py::arg("use_multicast") = true)
      .def("drop_multicast", [](PyHeap& h, int id) { h.heap->drop_multicast(id); })
      .def("get", [](PyHeap& h, int id) { return to_dict(h.heap->get(id)); })
      .def("release", [](PyHeap& h, int id) { h.heap->release(id); })
      // A tensor over rank `r`'s copy of allocation `id`.  It does not own the memory: keep the heap alive.
      .def("tensor", [](PyHeap& h, int id, int r, py::object dtype, int64_t numel) {
        const auto& a = h.heap->get(id);
        TORCH_CHECK(r >= 0 && r < (int)a.ptrs.size(), "SymmHeap.tensor: bad rank");
        const at::ScalarType st = torch::python::detail::py_object_to_dtype(dtype);
        TORCH_CHECK((size_t)numel * c10::elementSize(st) <= a.bytes, "SymmHeap.tensor: view exceeds the allocation");
        auto opt = at::TensorOptions().dtype(st);
        opt = h.host ? opt.device(at::kCPU) : opt.device(at::kCUDA, (c10::DeviceIndex)h.device);
        return at::from_blob(reinterpret_cast<void*>(a.ptrs[r]), {numel}, opt);
      });
}
