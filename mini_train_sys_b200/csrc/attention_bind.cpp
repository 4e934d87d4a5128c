#include <torch/extension.h>

void bind_attention(pybind11::module_& m) { (void)m; }
