// Host-only checks of llm::Tensor and the 16-bit codecs; the cases of the reference's
// tests/test_tensor.cpp:11-24 plus the view arithmetic the operators rely on.
#include "llm/tensor.h"

#include <cmath>
#include <iostream>
#include <stdexcept>
#include <string>

using namespace llm;

static void check(bool ok, const std::string& what) {
  if (!ok) throw std::runtime_error("test_tensor_host: " + what);
}
template <class F> static bool throws(F&& f) {
  try { f(); } catch (const std::exception&) { return true; }
  return false;
}

int main() {
  try {
    check(decode_f16(0x0001) == std::ldexp(1.f, -24), "half min subnormal");
    check(decode_f16(0x03ff) == std::ldexp(1.f, -14) - std::ldexp(1.f, -24), "half max subnormal");
    check(decode_f16(0x0400) == std::ldexp(1.f, -14), "half min normal");
    const float neg_zero = decode_f16(0x8000);
    check(neg_zero == 0 && std::signbit(neg_zero), "negative zero");
    check(std::isinf(decode_f16(0x7c00)) && !std::signbit(decode_f16(0x7c00)), "positive infinity");
    check(std::isnan(decode_f16(0x7e00)), "NaN");
    check(encode_f16(1.0f) == 0x3c00 && encode_f16(-2.0f) == 0xc000 && encode_f16(65504.0f) == 0x7bff, "encode exact values");
    check(encode_f16(1.0f + 3 * std::ldexp(1.f, -11)) == 0x3c01, "normals are truncated, as in the reference");
    check(encode_f16(1e9f) == 0x7c00 && encode_f16(std::ldexp(1.f, -24)) == 0x0001, "overflow / smallest subnormal");
    check(decode_bf16(encode_bf16(1.25f)) == 1.25f, "bf16 round trip");

    Tensor t = Tensor::from_f32({2, 3}, {1, 2, 3, 4, 5, 6});
    check(t.numel() == 6 && t.nbytes() == 24 && t.is_contiguous(), "numel / nbytes");
    check(t.strides() == std::vector<int64_t>({3, 1}), "row-major strides");
    Tensor r = t.reshape({3, 2});
    r.set_f32(0, 9);
    check(t.get_f32(0) == 9, "reshape shares storage");
    Tensor row1 = t.slice_first_dim(1, 1);
    check(row1.shape() == std::vector<int64_t>({1, 3}) && row1.storage_offset() == 12 && row1.get_f32(0) == 4, "slice_first_dim");
    check(t.prefix_first_dim(1).get_f32(2) == 3 && t.prefix_first_dim(1).storage_bytes() == 24, "prefix_first_dim");
    for (DType d : {DType::F16, DType::BF16}) {
      Tensor q(d, {2});
      q.set_f32(0, 1.25f);
      check(std::fabs(q.get_f32(0) - 1.25f) <= .02f, "dtype conversion");
    }
    Tensor ids(DType::I32, {3});
    ids.data_i32()[2] = 7;
    check(ids.data_i32()[2] == 7 && throws([&] { ids.get_f32(0); }) && throws([&] { ids.data_f32(); }), "I32 accessors");
    check(throws([] { Tensor bad(DType::F32, {-1}); }), "negative shape");
    check(throws([&] { t.reshape({4, 2}); }), "reshape element count");
    check(throws([&] { t.get_f32(6); }), "index bounds");
    check(throws([&] { t.slice_first_dim(2, 1); }) && throws([&] { t.prefix_first_dim(0); }), "slice bounds");
    check(Tensor().data() == nullptr && Tensor().numel() == 0, "default tensor");
    std::cout << "test_tensor_host passed\n";
    return 0;
  } catch (const std::exception& e) {
    std::cerr << e.what() << "\n";
    return 1;
  }
}
