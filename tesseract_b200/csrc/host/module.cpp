// pybind11 bindings of the host runtime (module name: _tsb_host).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <stdexcept>

#include "host_runtime.hpp"

namespace py = pybind11;
using namespace tsbh;

PYBIND11_MODULE(_tsb_host, m) {
  m.doc() = "tesseract_b200 host runtime: sampler, BPE merge loop, KV block allocator, parallel file reads";

  py::class_<HostSampler>(m, "HostSampler")
      .def(py::init([](float temperature, long long top_k, float top_p, float repetition_penalty, uint64_t seed) {
             SamplingParams p;
             p.temperature = temperature;
             p.top_k = top_k;
             p.top_p = top_p;
             p.repetition_penalty = repetition_penalty;
             return new HostSampler(p, seed);
           }),
           py::arg("temperature") = 1.f, py::arg("top_k") = 0, py::arg("top_p") = 1.f,
           py::arg("repetition_penalty") = 1.f, py::arg("seed") = 0)
      .def("reseed", &HostSampler::reseed)
      .def("next_u64", &HostSampler::next_u64)
      .def("uniform_double", &HostSampler::uniform_double)
      .def("sample",
           [](HostSampler& s, py::array_t<float, py::array::c_style | py::array::forcecast> logits,
              py::array_t<int64_t, py::array::c_style | py::array::forcecast> prev) {
             return s.sample(logits.data(), logits.size(), prev.data(), prev.size());
           },
           py::arg("logits"), py::arg("prev_tokens"));

  py::class_<BpeCore>(m, "BpeCore")
      .def(py::init<const std::unordered_map<std::string, int32_t>&, const std::vector<std::pair<std::string, std::string>>&,
                    const std::vector<std::string>&>())
      .def("encode_piece", [](const BpeCore& b, py::bytes piece) { return b.encode_piece(std::string(piece)); });

  py::class_<BlockAllocator>(m, "BlockAllocator")
      .def(py::init<int64_t>())
      .def("allocate", &BlockAllocator::allocate)
      .def("free", &BlockAllocator::free)
      .def("num_free", &BlockAllocator::num_free)
      .def("num_blocks", &BlockAllocator::num_blocks)
      .def("num_used", &BlockAllocator::num_used);

  m.def("read_ranges",
        [](const std::string& path, const std::vector<int64_t>& offsets, const std::vector<int64_t>& sizes,
           const std::vector<uintptr_t>& dst, int threads) {
          py::gil_scoped_release nogil;
          return read_ranges(path, offsets, sizes, dst, threads);
        },
        py::arg("path"), py::arg("offsets"), py::arg("sizes"), py::arg("dst"), py::arg("threads") = 8);
  m.def("safetensors_header", [](const std::string& path) {
    auto r = safetensors_header(path);
    return py::make_tuple(py::bytes(r.first), r.second);
  });
  m.def("token_mask",
        [](py::array_t<int32_t, py::array::c_style | py::array::forcecast> table, int32_t state, py::bytes all_bytes,
           py::array_t<int64_t, py::array::c_style | py::array::forcecast> offsets) {
          const std::string bytes(all_bytes);
          const int64_t n = offsets.size() - 1;
          py::array_t<uint8_t> out(n);
          token_mask(table.data(), table.shape(0), state, reinterpret_cast<const uint8_t*>(bytes.data()), offsets.data(), n,
                     out.mutable_data());
          return out;
        });

  m.def("compile_regex",
        [](py::bytes pattern, int64_t max_states) {
          const CompiledRegex r = compile_regex(std::string(pattern), max_states);
          const int64_t S = static_cast<int64_t>(r.accepting.size());
          py::array_t<int32_t> table({S, static_cast<int64_t>(256)});
          std::copy(r.table.begin(), r.table.end(), table.mutable_data());
          py::array_t<uint8_t> acc(S);
          std::copy(r.accepting.begin(), r.accepting.end(), acc.mutable_data());
          return py::make_tuple(table, acc, r.num_nfa_states);
        },
        py::arg("pattern"), py::arg("max_states") = 65536);

  m.def("gemm_avx2_supported", &gemm_avx2_supported);
  m.def("gemm_num_threads", &gemm_num_threads, py::arg("M"), py::arg("N"), py::arg("K"), py::arg("requested") = 0);
  m.def("gemm_f32",
        [](py::array_t<float, py::array::c_style | py::array::forcecast> A,
           py::array_t<float, py::array::c_style | py::array::forcecast> B, bool b_nk, int threads) {
          if (A.ndim() != 2 || B.ndim() != 2) throw std::invalid_argument("gemm_f32: A and B must be matrices");
          const int64_t M = A.shape(0), K = A.shape(1);
          const int64_t N = b_nk ? B.shape(0) : B.shape(1);
          if ((b_nk ? B.shape(1) : B.shape(0)) != K) throw std::invalid_argument("gemm_f32: inner dimensions differ");
          py::array_t<float> C({M, N});
          {
            py::gil_scoped_release nogil;
            gemm_f32(A.data(), K, B.data(), B.shape(1), b_nk, C.mutable_data(), N, M, N, K, threads);
          }
          return C;
        },
        py::arg("A"), py::arg("B"), py::arg("b_nk") = false, py::arg("threads") = 0);
  m.def("gemv_vnni_supported", &gemv_vnni_supported);
  m.def("quantize_row_int8", [](py::array_t<float, py::array::c_style | py::array::forcecast> x) {
    py::array_t<int8_t> q(x.size());
    const float scale = quantize_row_int8(x.data(), x.size(), q.mutable_data());
    return py::make_tuple(q, scale);
  });
  m.def("compute_row_sums", [](py::array_t<int8_t, py::array::c_style | py::array::forcecast> W) {
    if (W.ndim() != 2) throw std::invalid_argument("compute_row_sums: W must be [N, K]");
    py::array_t<int32_t> out(W.shape(0));
    compute_row_sums(W.data(), W.shape(0), W.shape(1), out.mutable_data());
    return out;
  });
  m.def("gemv_w8a8",
        [](py::array_t<int8_t, py::array::c_style | py::array::forcecast> W,
           py::array_t<float, py::array::c_style | py::array::forcecast> wscale, py::object rowsum,
           py::array_t<int8_t, py::array::c_style | py::array::forcecast> xq, float xscale, int64_t n_begin, int64_t n_end,
           int threads) {
          if (W.ndim() != 2) throw std::invalid_argument("gemv_w8a8: W must be [N, K]");
          const int64_t N = W.shape(0), K = W.shape(1);
          if (wscale.size() != N || xq.size() != K) throw std::invalid_argument("gemv_w8a8: wscale [N] and xq [K] expected");
          if (n_end < 0) n_end = N;
          if (n_begin < 0 || n_end > N || n_begin > n_end) throw std::invalid_argument("gemv_w8a8: bad row range");
          py::array_t<int32_t, py::array::c_style | py::array::forcecast> rs;
          const int32_t* rsp = nullptr;
          if (!rowsum.is_none()) {
            rs = rowsum.cast<py::array_t<int32_t, py::array::c_style | py::array::forcecast>>();
            if (rs.size() != N) throw std::invalid_argument("gemv_w8a8: rowsum [N] expected");
            rsp = rs.data();
          }
          py::array_t<float> y(N);
          float* yp = y.mutable_data();
          std::fill(yp, yp + N, 0.f);
          {
            py::gil_scoped_release nogil;
            if (n_begin == 0 && n_end == N)
              gemv_w8a8(W.data(), wscale.data(), rsp, xq.data(), xscale, yp, N, K, threads);
            else
              gemv_w8a8_range(W.data(), wscale.data(), rsp, xq.data(), xscale, yp, n_begin, n_end, K);
          }
          return y;
        },
        py::arg("W"), py::arg("wscale"), py::arg("rowsum"), py::arg("xq"), py::arg("xscale"), py::arg("n_begin") = 0,
        py::arg("n_end") = -1, py::arg("threads") = 0);
}
