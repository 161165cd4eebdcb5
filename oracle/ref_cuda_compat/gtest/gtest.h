// A few lines standing in for googletest (the reference's submodule is empty): enough
// to compile and run the reference's tests/cpp known-answer tests.  A failed assertion
// prints where and what, marks the test failed and returns from the test body.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

namespace kat {
struct Case {
  const char *suite, *name;
  void (*fn)();
};
inline std::vector<Case> &cases() {
  static std::vector<Case> v;
  return v;
}
inline int &failures() {
  static int n = 0;
  return n;
}
struct Registrar {
  Registrar(const char *s, const char *n, void (*f)()) { cases().push_back(Case{s, n, f}); }
};
// swallows the `<< "message"` tail of a failed assertion and prints it
struct Fail {
  std::ostringstream os;
  Fail(const char *file, int line, const std::string &what) {
    ++failures();
    os << file << ":" << line << ": " << what << " ";
  }
  template <typename T>
  Fail &operator<<(const T &v) {
    os << v;
    return *this;
  }
  ~Fail() { std::cerr << os.str() << std::endl; }
};
struct Void {
  void operator=(const Fail &) {}
};
// googletest's "almost equal": within 4 units in the last place
template <typename F, typename I>
inline bool almost_equal(F a, F b) {
  if (std::isnan(a) || std::isnan(b)) return false;
  if (a == b) return true;
  I ia, ib;
  std::memcpy(&ia, &a, sizeof a);
  std::memcpy(&ib, &b, sizeof b);
  const I sign = I(1) << (sizeof(I) * 8 - 1);
  auto biased = [&](I v) { return (v & sign) ? I(~v + 1) : I(v | sign); };
  const I x = biased(ia), y = biased(ib);
  return (x > y ? x - y : y - x) <= 4;
}
template <typename A, typename B>
inline std::string show(const char *ea, const char *eb, const A &a, const B &b) {
  std::ostringstream os;
  os << "expected " << ea << " == " << eb << ", got " << +a << " vs " << +b;
  return os.str();
}
}  // namespace kat

#define TEST(suite, name)                                                        \
  static void kat_##suite##_##name();                                            \
  static kat::Registrar kat_reg_##suite##_##name(#suite, #name, kat_##suite##_##name); \
  static void kat_##suite##_##name()

#define KAT_CHECK(ok, what) \
  if (ok) {                 \
  } else                    \
    return kat::Void() = kat::Fail(__FILE__, __LINE__, what)

#define ASSERT_EQ(a, b) KAT_CHECK((a) == (b), kat::show(#a, #b, (a), (b)))
#define ASSERT_FLOAT_EQ(a, b) \
  KAT_CHECK((kat::almost_equal<float, uint32_t>(float(a), float(b))), kat::show(#a, #b, float(a), float(b)))
#define ASSERT_DOUBLE_EQ(a, b) \
  KAT_CHECK((kat::almost_equal<double, uint64_t>(double(a), double(b))), kat::show(#a, #b, double(a), double(b)))
