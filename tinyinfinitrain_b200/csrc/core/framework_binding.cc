// Python bindings of the C++ framework facade (Tensor / autograd::Function / nn / optimizers).
#include <torch/extension.h>

void bind_framework(pybind11::module_& m) { (void)m; }
