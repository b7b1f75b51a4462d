// Python bindings of the attention kernels (flash_attn.cu).
#include <torch/extension.h>

void ody_register_attention(pybind11::module& m) { (void)m; }
