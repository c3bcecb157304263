// Python module q8_1_me: same functions and argument order as the reference's
// src/bindings/q8_1_binding.cpp:11-44 (quantize(input, output, dims) writes in place,
// parse(raw, n_blocks) -> (qs, scale, sum)).  Where the reference silently copies an array of
// the wrong dtype (and so loses the output), this module raises.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "../../../include/jq_b200.h"

namespace py = pybind11;

static void raise_on(int rc, const char *who) {
    if (rc == JQ_OK) return;
    const std::string msg = std::string(who) + ": " + jq_last_error();
    if (rc == JQ_ERR_INVALID_ARG || rc == JQ_ERR_SHAPE || rc == JQ_ERR_ALIGN) throw py::value_error(msg);
    throw std::runtime_error(msg);
}

PYBIND11_MODULE(q8_1_me, m) {
    m.doc() = "Q8_1 (block_q8_1_mmq) activation quantizer for sm_100a";
    m.def(
        "quantize",
        [](py::array input, py::array output, std::vector<int> dims) {
            if (!py::isinstance<py::array_t<float>>(input)) throw py::value_error("quantize: input must be float32");
            if (!py::isinstance<py::array_t<uint8_t>>(output)) throw py::value_error("quantize: output must be uint8");
            if (!(input.flags() & (py::array::c_style | py::array::f_style)))
                throw py::value_error("quantize: input must be contiguous");
            if (!(output.flags() & py::array::c_style) || !output.writeable())
                throw py::value_error("quantize: output must be a writeable C-contiguous array");
            int64_t n = 1, m_cols = 1;
            for (size_t i = 0; i < dims.size(); ++i) {
                n *= dims[i];
                if (i > 0) m_cols *= dims[i];
            }
            if (dims.empty() || (int64_t)input.size() < n) throw py::value_error("quantize: dims exceed the input size");
            if ((size_t)output.nbytes() < jq_q8_1_bytes(dims[0], m_cols))
                throw py::value_error("quantize: output buffer too small");
            raise_on(jq_q8_1_host(static_cast<const float *>(input.data()), static_cast<uint8_t *>(output.mutable_data()),
                                  dims.data(), (int)dims.size()),
                     "quantize");
        },
        py::arg("input"), py::arg("output"), py::arg("dims"), "Quantize float32 to Q8_1");

    m.def(
        "parse",
        [](py::array_t<uint8_t, py::array::c_style | py::array::forcecast> raw, int64_t n_blocks) {
            if (n_blocks < 0 || (int64_t)raw.size() < n_blocks * 144) throw py::value_error("parse: raw buffer too small");
            py::array_t<int8_t> qs({(py::ssize_t)n_blocks, (py::ssize_t)128});
            py::array_t<float> scale({(py::ssize_t)n_blocks, (py::ssize_t)4});
            py::array_t<float> sum({(py::ssize_t)n_blocks, (py::ssize_t)4});
            raise_on(jq_parse_q8_1_output(raw.data(), qs.mutable_data(), scale.mutable_data(), sum.mutable_data(), n_blocks),
                     "parse");
            return py::make_tuple(qs, scale, sum);
        },
        py::arg("raw"), py::arg("n_blocks"), "Parse raw Q8_1 output");
}
