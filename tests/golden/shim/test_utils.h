// Shadows the reference's src/tim/vx/test_utils.h for the golden-fixture
// harness: it pulls in that header unchanged (quantization helpers the tests
// use to build their vectors) but routes ArraysMatch through a wrapper that
// also hands the expected vector and its tolerance to the capture hook.
#ifndef GOLDEN_SHIM_TEST_UTILS_H_
#define GOLDEN_SHIM_TEST_UTILS_H_

#include <sys/types.h>
#include "gtest/gtest.h"

#define ArraysMatch ArraysMatchElementwise
#include REFERENCE_TEST_UTILS_H
#undef ArraysMatch

namespace {
template <typename T>
::testing::AssertionResult ArraysMatch(const std::vector<T>& expected, const std::vector<T>& actual, T abs_error) {
  if (expected.size() == actual.size() && ::testing::internal::dtype_code<T>::value)
    orc_capture_expect_pair(expected.data(), actual.data(), expected.size() * sizeof(T),
                            ::testing::internal::dtype_code<T>::value, static_cast<double>(abs_error));
  return ArraysMatchElementwise(expected, actual, abs_error);
}
template <typename T>
::testing::AssertionResult ArraysMatch(const std::vector<T>& expected, const std::vector<T>& actual, T abs_error,
                                       const std::string& msg) {
  if (expected.size() == actual.size() && ::testing::internal::dtype_code<T>::value)
    orc_capture_expect_pair(expected.data(), actual.data(), expected.size() * sizeof(T),
                            ::testing::internal::dtype_code<T>::value, static_cast<double>(abs_error));
  return ArraysMatchElementwise(expected, actual, abs_error, msg);
}
}  // namespace
#endif  // GOLDEN_SHIM_TEST_UTILS_H_
