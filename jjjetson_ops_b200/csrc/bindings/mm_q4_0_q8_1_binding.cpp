// Python module mm_q4_0_q8_1_me: same function, argument order and keyword names as the
// reference's src/bindings/mm_q4_0_q8_1_binding.cpp:13-22.  One optional keyword is added
// (s_mode, default 0 = the reference's s = sum(x)).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "../../../include/jq_b200.h"

namespace py = pybind11;

PYBIND11_MODULE(mm_q4_0_q8_1_me, m) {
    m.doc() = "Q4_0 x Q8_1 quantized multiply for sm_100a";
    m.def(
        "mmq",
        [](py::array weight, py::array input, py::array quant_buf, py::array output, std::vector<int> input_dims,
           int nrows_out, int ncols_k, int s_mode) {
            if (!py::isinstance<py::array_t<uint8_t>>(weight) || !py::isinstance<py::array_t<uint8_t>>(quant_buf))
                throw py::value_error("mmq: weight_q4_0 and quant_workspace must be uint8");
            if (!py::isinstance<py::array_t<float>>(input) || !py::isinstance<py::array_t<float>>(output))
                throw py::value_error("mmq: input and output must be float32");
            if (!(weight.flags() & py::array::c_style) || !(quant_buf.flags() & py::array::c_style) ||
                !(input.flags() & (py::array::c_style | py::array::f_style)) ||
                !(output.flags() & (py::array::c_style | py::array::f_style)))
                throw py::value_error("mmq: arrays must be contiguous");
            if (!quant_buf.writeable() || !output.writeable())
                throw py::value_error("mmq: quant_workspace and output must be writeable");
            int64_t batch = 1;
            for (size_t i = 1; i < input_dims.size(); ++i) batch *= input_dims[i];
            if (input_dims.size() < 2) throw py::value_error("mmq: input_dims needs at least [K, batch]");
            if ((size_t)weight.nbytes() < jq_q4_0_bytes(nrows_out, ncols_k)) throw py::value_error("mmq: weight buffer too small");
            if ((int64_t)input.size() < (int64_t)ncols_k * batch) throw py::value_error("mmq: input too small");
            if ((size_t)quant_buf.nbytes() < jq_q8_1_bytes(ncols_k, batch)) throw py::value_error("mmq: quant_workspace too small");
            if ((int64_t)output.size() < (int64_t)nrows_out * batch) throw py::value_error("mmq: output too small");
            const int rc = jq_mat_mul_q4_0_q8_1_host_ex(weight.data(), static_cast<const float *>(input.data()),
                                                        static_cast<uint8_t *>(quant_buf.mutable_data()),
                                                        static_cast<float *>(output.mutable_data()), input_dims.data(),
                                                        (int)input_dims.size(), nrows_out, ncols_k, s_mode);
            if (rc != JQ_OK) {
                const std::string msg = std::string("mmq: ") + jq_last_error();
                if (rc == JQ_ERR_INVALID_ARG || rc == JQ_ERR_SHAPE || rc == JQ_ERR_ALIGN) throw py::value_error(msg);
                throw std::runtime_error(msg);
            }
        },
        py::arg("weight_q4_0"), py::arg("input"), py::arg("quant_workspace"), py::arg("output"), py::arg("input_dims"),
        py::arg("nrows_out"), py::arg("ncols_k"), py::arg("s_mode") = 0,
        "Q4_0 weight x float activation (quantize via q8_1) -> float output");
}
