// Minimal stand-in for GoogleTest, just large enough to compile and run the
// reference's own *_test.cc files against this repository's tim::vx API when
// producing golden fixtures (GoogleTest itself is not installed here).
// Besides checking, vector comparisons are forwarded to the oracle backend's
// capture hook so the expected values end up in the fixture files.
#ifndef GOLDEN_SHIM_GTEST_H_
#define GOLDEN_SHIM_GTEST_H_

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <sstream>
#include <string>
#include <type_traits>
#include <vector>

extern "C" void orc_capture_set_case(const char* name);
extern "C" void orc_capture_expect_pair(const void* a, const void* b, size_t bytes, int32_t dtype, double tol);

namespace testing {

namespace internal {
struct TestInfo {
  const char* suite;
  const char* name;
  void (*body)();
};
std::vector<TestInfo>& registry();
int& failure_count();
bool& skipped();
struct Registrar {
  Registrar(const char* s, const char* n, void (*b)()) { registry().push_back({s, n, b}); }
};

template <typename T> struct dtype_code { static const int32_t value = 0; };
template <> struct dtype_code<int8_t> { static const int32_t value = 1; };
template <> struct dtype_code<uint8_t> { static const int32_t value = 2; };
template <> struct dtype_code<int32_t> { static const int32_t value = 5; };
template <> struct dtype_code<float> { static const int32_t value = 9; };

// Result of one assertion; swallows anything streamed into it and prints it on failure.
class Result {
 public:
  Result(bool ok, const char* file, int line, const std::string& what) : ok_(ok) {
    if (!ok_) {
      ++failure_count();
      msg_ << file << ":" << line << ": Failure: " << what << " ";
    }
  }
  Result(const Result& o) : ok_(o.ok_) { msg_ << o.msg_.str(); const_cast<Result&>(o).ok_ = true; }
  ~Result() { if (!ok_) std::cerr << msg_.str() << std::endl; }
  template <typename T> Result& operator<<(const T& v) { if (!ok_) msg_ << v; return *this; }
  explicit operator bool() const { return ok_; }
 private:
  bool ok_;
  std::ostringstream msg_;
};

template <typename T> std::string show(const T& v) { std::ostringstream s; s << v; return s.str(); }
inline std::string show(const uint8_t& v) { return std::to_string(static_cast<int>(v)); }
inline std::string show(const int8_t& v) { return std::to_string(static_cast<int>(v)); }
template <typename T> std::string show(const std::vector<T>& v) {
  std::ostringstream s;
  s << "{";
  for (size_t i = 0; i < v.size() && i < 32; ++i) s << (i ? ", " : "") << show(v[i]);
  if (v.size() > 32) s << ", ...";
  s << "}";
  return s.str();
}

template <typename A, typename B>
Result expect_eq(const A& a, const B& b, const char* ea, const char* eb, const char* file, int line) {
  bool ok = (a == b);
  return Result(ok, file, line, ok ? "" : std::string(ea) + " == " + eb + " (" + show(a) + " vs " + show(b) + ")");
}
template <typename T>
Result expect_eq(const std::vector<T>& a, const std::vector<T>& b, const char* ea, const char* eb, const char* file, int line) {
  if (a.size() == b.size() && dtype_code<T>::value)
    orc_capture_expect_pair(a.data(), b.data(), a.size() * sizeof(T), dtype_code<T>::value, 0.0);
  bool ok = (a == b);
  return Result(ok, file, line, ok ? "" : std::string(ea) + " == " + eb + " (" + show(a) + " vs " + show(b) + ")");
}
template <typename A, typename B, typename C>
Result expect_near(const A& a, const B& b, const C& tol, const char* file, int line) {
  double d = std::fabs(static_cast<double>(a) - static_cast<double>(b));
  bool ok = d <= static_cast<double>(tol);
  return Result(ok, file, line, ok ? "" : "|" + show(a) + " - " + show(b) + "| > " + show(tol));
}
}  // namespace internal

class AssertionResult {
 public:
  explicit AssertionResult(bool ok) : ok_(ok) {}
  operator bool() const { return ok_; }
  template <typename T> AssertionResult& operator<<(const T&) { return *this; }
 private:
  bool ok_;
};
inline AssertionResult AssertionSuccess() { return AssertionResult(true); }
inline AssertionResult AssertionFailure() { return AssertionResult(false); }

class Test {};

}  // namespace testing

#define TEST(suite, name)                                                                  \
  static void suite##_##name##_body();                                                     \
  static ::testing::internal::Registrar suite##_##name##_reg(#suite, #name, &suite##_##name##_body); \
  static void suite##_##name##_body()

#define EXPECT_TRUE(c) ::testing::internal::Result(static_cast<bool>(c), __FILE__, __LINE__, #c " is false")
#define EXPECT_FALSE(c) ::testing::internal::Result(!static_cast<bool>(c), __FILE__, __LINE__, #c " is true")
#define EXPECT_EQ(a, b) ::testing::internal::expect_eq((a), (b), #a, #b, __FILE__, __LINE__)
#define EXPECT_NE(a, b) ::testing::internal::Result(!((a) == (b)), __FILE__, __LINE__, #a " != " #b)
#define EXPECT_NEAR(a, b, tol) ::testing::internal::expect_near((a), (b), (tol), __FILE__, __LINE__)
#define EXPECT_FLOAT_EQ(a, b) ::testing::internal::expect_near((a), (b), 4e-7 * (std::fabs(static_cast<double>(a)) + 1e-30), __FILE__, __LINE__)
#define ASSERT_TRUE(c) if (!(c)) { ::testing::internal::Result(false, __FILE__, __LINE__, #c " is false"); return; } else (void)0
#define ASSERT_EQ(a, b) if (!((a) == (b))) { ::testing::internal::Result(false, __FILE__, __LINE__, #a " == " #b); return; } else (void)0
#define GTEST_SKIP() do { ::testing::internal::skipped() = true; return; } while (0)

#endif  // GOLDEN_SHIM_GTEST_H_
