// pybind11 / libtorch module `mixedgemm`: the drop-in for the module MixedGemm builds from
// its src/bindings.cpp (entry points at :311-342 there, consumed by its main.py:35,36,59).
// Same function names, keyword names, positional order, tensor shapes and dtypes; torch is
// used for tensor ownership and the current stream only - all work goes through the C ABI
// of libmixedgemm_b200 (include/mixedgemm_c.h).
//
// Deliberate differences: any K whose segments are multiples of 32 is accepted (the
// reference dispatches seven compile-time K values, :95-168); inputs are validated (the
// reference's checks are commented out, :24-29); nothing synchronises or prints
// (:51-65 does); scale buffers are sized for whole 512-byte atoms when that is larger
// than the reference's (M/128+1)*128*K/32; the GEMM result buffer is not zero-filled first.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <algorithm>
#include <string>
#include <tuple>

#include "mixedgemm_c.h"

namespace {

void check(int status, const char* where) {
  if (status == MG_OK) return;
  std::string msg = std::string(where) + ": " + mg_strerror(status);
  if (status == MG_ERR_CUDA) msg += " (cudaError " + std::to_string(mg_last_cuda_error()) + ")";
  throw std::runtime_error(msg);
}

uint8_t* u8(const torch::Tensor& t) { return t.numel() ? t.data_ptr<uint8_t>() : nullptr; }

// Code tensors may be row-pitched views (what the quantisers of this module return); scale
// tensors are flat.
void check_u8(const torch::Tensor& t, const char* name, bool codes) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kUInt8, "matmul: ", name, " must be a CUDA uint8 tensor");
  if (codes) {
    TORCH_CHECK(t.dim() == 2 && (t.size(1) == 0 || t.stride(1) == 1), "matmul: ", name,
                " must be 2-D with unit column stride");
  } else {
    TORCH_CHECK(t.is_contiguous(), "matmul: ", name, " must be contiguous");
  }
}

size_t pitch_of(const torch::Tensor& t) { return t.size(1) ? (size_t)t.stride(0) : 0; }

using Six = std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor>;

torch::Tensor matmul(const torch::Tensor& AN, const torch::Tensor& BN, const torch::Tensor& AS,
                     const torch::Tensor& BS, const torch::Tensor& AO, const torch::Tensor& BO,
                     const torch::Tensor& SFAN, const torch::Tensor& SFBN, const torch::Tensor& SFAS,
                     const torch::Tensor& SFBS, const torch::Tensor& SFAO, const torch::Tensor& SFBO) {
  const torch::Tensor* all[] = {&AN, &BN, &AS, &BS, &AO, &BO, &SFAN, &SFBN, &SFAS, &SFBS, &SFAO, &SFBO};
  const char* names[] = {"AN", "BN", "AS", "BS", "AO", "BO", "SFAN", "SFBN", "SFAS", "SFBS", "SFAO", "SFBO"};
  for (int i = 0; i < 12; ++i) check_u8(*all[i], names[i], i < 6);
  // shape inference as in the reference (src/bindings.cpp:30-34)
  const int M = (int)AN.size(0), N = (int)BN.size(0);
  const int KN = (int)AN.size(1) * 2, KS = (int)(AS.size(1) * 4 / 3), KO = (int)AO.size(1);
  // The reference infers the sizes from AN, BN, AS and AO and trusts the rest; the tensor maps and
  // the whole-atom scale copies are built from these sizes, so every other tensor is held to them.
  TORCH_CHECK(AS.size(0) == M && AO.size(0) == M, "matmul: AS and AO must have AN's row count");
  TORCH_CHECK(BS.size(0) == N && BO.size(0) == N, "matmul: BS and BO must have BN's row count");
  TORCH_CHECK(AS.size(1) * 4 == (int64_t)KS * 3, "matmul: AS must hold 3 bytes per 4 elements");
  TORCH_CHECK(BN.size(1) * 2 == KN && BS.size(1) * 2 == KS && BO.size(1) * 2 == KO,
              "matmul: weight code widths do not match the activation segments");
  const torch::Tensor* sfs[] = {&SFAN, &SFBN, &SFAS, &SFBS, &SFAO, &SFBO};
  const int sf_rows[] = {M, N, M, N, M, N}, sf_k[] = {KN, KN, KS, KS, KO, KO};
  for (int i = 0; i < 6; ++i)
    TORCH_CHECK((size_t)sfs[i]->numel() >= mg_sf_bytes(sf_rows[i], sf_k[i]), "matmul: ", names[6 + i], " holds ",
                sfs[i]->numel(), " bytes, ", mg_sf_bytes(sf_rows[i], sf_k[i]),
                " are read (whole 512-byte atoms of 128 rows x 128 elements)");
  for (int i = 1; i < 12; ++i)
    TORCH_CHECK(all[i]->device() == AN.device(), "matmul: ", names[i], " is on another device than AN");
  c10::cuda::CUDAGuard guard(AN.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto C = torch::empty({M, N}, torch::dtype(torch::kBFloat16).device(AN.device()));
  const size_t pitches[6] = {pitch_of(AN), pitch_of(BN), pitch_of(AS), pitch_of(BS), pitch_of(AO), pitch_of(BO)};
  const size_t wsb = mg_matmul_pitched_workspace_bytes(M, N, KN, KS, KO, pitches);
  torch::Tensor ws;
  uint8_t* wsp = nullptr;
  if (wsb) {
    ws = torch::empty({(int64_t)wsb + 1024}, torch::dtype(torch::kUInt8).device(AN.device()));
    wsp = ws.data_ptr<uint8_t>();
    wsp += (1024 - reinterpret_cast<uintptr_t>(wsp) % 1024) % 1024;
  }
  check(mg_matmul_pitched(u8(AN), u8(BN), u8(AS), u8(BS), u8(AO), u8(BO), pitches, 0, M, N, KN, KS, KO, nullptr,
                          C.data_ptr(), N, u8(SFAN), u8(SFBN), u8(SFAS), u8(SFBS), u8(SFAO), u8(SFBO), wsp, wsb,
                          stream.stream()),
        "matmul");
  return C;
}

Six reorder_quantize(bool weights, const torch::Tensor& X, const torch::Tensor& reorder_index, int KN, int KS, int KO) {
  const char* where = weights ? "reorder_quantize_w" : "reorder_quantize_x";
  TORCH_CHECK(X.is_cuda() && X.scalar_type() == torch::kBFloat16 && X.dim() == 2 && X.is_contiguous(), where,
              ": expected a contiguous 2-D CUDA bfloat16 tensor");
  TORCH_CHECK(reorder_index.is_cuda() && reorder_index.scalar_type() == torch::kInt16 && reorder_index.is_contiguous(),
              where, ": reorder_index must be a contiguous CUDA int16 tensor");
  const int R = (int)X.size(0), K = (int)X.size(1);
  if (K != KN + KS + KO || reorder_index.numel() != K) {
    // the reference throws std::runtime_error for a K it does not know (src/bindings.cpp:165-168)
    throw std::runtime_error(std::string("Value error in ") + where + ": K does not match KN+KS+KO");
  }
  c10::cuda::CUDAGuard guard(X.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto o = torch::dtype(torch::kUInt8).device(X.device());
  auto sf_len = [&](int k) {
    const int64_t ref = weights ? (int64_t)R * k / 32 : (int64_t)(R / 128 + 1) * 128 * k / 32;
    return std::max<int64_t>(ref, (int64_t)mg_sf_bytes(R, k));
  };
  // the reference's shapes, as views of buffers whose row pitch the GEMM can read in place
  auto codes = [&](int seg, int64_t logical, int k) {
    const int64_t pitch = (int64_t)mg_code_pitch(weights, seg, k);
    auto buf = torch::empty({R, pitch}, o);
    return pitch == logical ? buf : buf.narrow(1, 0, logical);
  };
  auto c4 = codes(0, KN / 2, KN);
  auto c6 = codes(1, weights ? KS / 2 : KS / 4 * 3, KS);
  auto c8 = codes(2, weights ? KO / 2 : KO, KO);
  auto s4 = torch::empty({sf_len(KN)}, o), s6 = torch::empty({sf_len(KS)}, o), s8 = torch::empty({sf_len(KO)}, o);
  const size_t pitches[3] = {pitch_of(c4), pitch_of(c6), pitch_of(c8)};
  check(mg_reorder_quantize_pitched(weights, X.data_ptr(), R, K, reorder_index.data_ptr<int16_t>(), KN, KS, KO, u8(c4),
                                    u8(c6), u8(c8), pitches, u8(s4), u8(s6), u8(s8), stream.stream()),
        where);
  return std::make_tuple(c4, c6, c8, s4, s6, s8);
}

Six reorder_quantize_x(const torch::Tensor& X, const torch::Tensor& reorder_index, const int KN, const int KS,
                       const int KO, const int seqlen, const int outfeatures) {
  (void)seqlen;
  (void)outfeatures;
  return reorder_quantize(false, X, reorder_index, KN, KS, KO);
}

Six reorder_quantize_w(const torch::Tensor& W, const torch::Tensor& reorder_index, const int KN, const int KS,
                       const int KO, const int seqlen, const int outfeatures) {
  (void)seqlen;
  (void)outfeatures;
  return reorder_quantize(true, W, reorder_index, KN, KS, KO);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("matmul", &matmul,
        "input: AN (M x KN/2), BN (N x KN/2), AS (M x 3KS/4), BS (N x KS/2), AO (M x KO), BO (N x KO/2), "
        "SFAN, SFBN, SFAS, SFBS, SFAO, SFBO: uint8 CUDA tensors\n"
        "output: torch.Tensor(M x N, BFLOAT16, CUDA) = A @ B^T",
        py::arg("AN"), py::arg("BN"), py::arg("AS"), py::arg("BS"), py::arg("AO"), py::arg("BO"), py::arg("SFAN"),
        py::arg("SFBN"), py::arg("SFAS"), py::arg("SFBS"), py::arg("SFAO"), py::arg("SFBO"));
  m.def("test_function", []() { return "Hello from test_function!"; });
  m.def("reorder_quantize_x", &reorder_quantize_x, "Reorder and quantize activation", py::arg("X"),
        py::arg("reorder_index"), py::arg("KN"), py::arg("KS"), py::arg("KO"), py::arg("seqlen"),
        py::arg("outfeatures"));
  m.def("reorder_quantize_w", &reorder_quantize_w, "Reorder and quantize weight", py::arg("W"),
        py::arg("reorder_index"), py::arg("KN"), py::arg("KS"), py::arg("KO"), py::arg("seqlen"),
        py::arg("outfeatures"));
}
