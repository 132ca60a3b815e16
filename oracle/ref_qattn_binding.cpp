// One-function binding of the reference's attention extension, used only by oracle/build_ref.py:
// qk_int8_sv_f16_accum_f16_attn is declared in the reference's csrc/qattn/attn_cuda_sm80.h:19-30 and
// defined in csrc/qattn/qk_int_sv_f16_cuda_sm80.cu:905-1080.  (The reference's own pybind_sm80.cpp binds
// three more functions from a second source file that the processors do not call.)
#include <torch/extension.h>

#include "attn_cuda_sm80.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("qk_int8_sv_f16_accum_f16_attn", &qk_int8_sv_f16_accum_f16_attn, "int8 QK^T, fp16 PV, fp16 accumulation");
}
