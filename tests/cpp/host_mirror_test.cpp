// Exercises include/xnq.hpp (the C++ host mirror of xn's quantized operator API).
//   host_mirror_test cpu                      shape / dtype errors that need no device
//   host_mirror_test gpu <dtype> <n> <k> <m> <weights.bin> <x.bin> <bias.bin> <y_out.bin>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>

#include "xnq.hpp"

static std::vector<uint8_t> read_all(const char *path) {
  std::ifstream f(path, std::ios::binary);
  return std::vector<uint8_t>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}
template <typename F>
static bool throws(F f, const char *needle) {
  try {
    f();
  } catch (const xnq::Error &e) {
    if (std::string(e.what()).find(needle) != std::string::npos) return true;
    std::cerr << "unexpected message: " << e.what() << "\n";
    return false;
  }
  std::cerr << "no exception (wanted '" << needle << "')\n";
  return false;
}

int main(int argc, char **argv) {
  using namespace xnq;
  if (argc >= 2 && std::string(argv[1]) == "cpu") {
    bool ok = true;
    ok &= type_size(GgmlDType::Q4_0) == 18 && type_size(GgmlDType::Q8_0) == 34 && type_size(GgmlDType::Q4K) == 144 && type_size(GgmlDType::Q6K) == 210;
    ok &= block_size(GgmlDType::Q4_0) == 32 && block_size(GgmlDType::Q6K) == 256;
    ok &= throws([] { QTensor(std::vector<uint8_t>(18), {1, 33}, GgmlDType::Q4_0); }, "divisible by block size");
    ok &= throws([] { QTensor(std::vector<uint8_t>(), {}, GgmlDType::Q4_0); }, "scalar tensor");
    ok &= throws([] { QTensor(std::vector<uint8_t>(70), {4, 32}, GgmlDType::Q4_0); }, "wants 72 bytes");
    QTensor qt(std::vector<uint8_t>(72), {4, 32}, GgmlDType::Q4_0);
    ok &= qt.rank() == 2 && qt.storage_size_in_bytes() == 72 && qt.dtype() == GgmlDType::Q4_0;
    ok &= throws([&] { Q80::linear_from_qtensor(qt, 32, 4); }, "expected a Q8_0 tensor");
    ok &= throws([&] { Q40::linear_from_qtensor(qt, 32, 8); }, "expected [8, 32]");
    std::puts(ok ? "cpu ok" : "cpu FAILED");
    return ok ? 0 : 1;
  }
  if (argc == 10 && std::string(argv[1]) == "gpu") {
    const GgmlDType dt = (GgmlDType)std::atoi(argv[2]);
    const int64_t n = std::atoll(argv[3]), k = std::atoll(argv[4]), m = std::atoll(argv[5]);
    try {
      check(xnq_init(0));
      QTensor qt(read_all(argv[6]), {n, k}, dt);
      auto xb = read_all(argv[7]), bb = read_all(argv[8]);
      std::vector<float> bias((const float *)bb.data(), (const float *)bb.data() + bb.size() / 4);
      QCudaTensor w = QCudaTensor::from_qtensor(qt);
      if (w.data() != qt.data()) {
        std::puts("canonical bytes differ");
        return 1;
      }
      QCudaLinear lin(std::move(w), bias);
      std::vector<float> y((size_t)m * n);
      const auto od = lin.forward_host((const float *)xb.data(), {m / 2, 2, k}, y.data());   // a 3-d input, as qlinear_3d_input
      if (od.size() != 3 || od[0] != m / 2 || od[1] != 2 || od[2] != n) return 1;
      if (!throws([&] { lin.forward_host((const float *)xb.data(), {k}, y.data()); }, "only one dimension")) return 1;
      if (!throws([&] { lin.forward_host((const float *)xb.data(), {m, k + 32}, y.data()); }, "incompatible with")) return 1;
      std::ofstream(argv[9], std::ios::binary).write((const char *)y.data(), (std::streamsize)(y.size() * 4));
      std::puts("gpu ok");
      return 0;
    } catch (const Error &e) {
      std::cerr << "xnq error " << e.code << ": " << e.what() << "\n";
      return 2;
    }
  }
  std::fputs("usage: host_mirror_test cpu | gpu <dtype> <n> <k> <m> <weights> <x> <bias> <y_out>\n", stderr);
  return 64;
}
