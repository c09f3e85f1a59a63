// Runner for the GoogleTest stand-in: each test runs in its own child process
// so that one crashing case cannot take the rest down.  Prints one line per
// test: "OK|FAIL|SKIP|CRASH|DISABLED Suite.name".
#include <sys/wait.h>
#include <unistd.h>

#include <cstring>

#include "gtest/gtest.h"

namespace testing {
namespace internal {
std::vector<TestInfo>& registry() { static std::vector<TestInfo> r; return r; }
int& failure_count() { static int n = 0; return n; }
bool& skipped() { static bool s = false; return s; }
}  // namespace internal
}  // namespace testing

int main() {
  int bad = 0;
  for (const auto& t : ::testing::internal::registry()) {
    std::string full = std::string(t.suite) + "." + t.name;
    if (std::strncmp(t.name, "DISABLED_", 9) == 0) {
      std::printf("DISABLED %s\n", full.c_str());
      continue;
    }
    std::fflush(stdout);
    pid_t pid = fork();
    if (pid == 0) {
      orc_capture_set_case(full.c_str());
      t.body();
      std::fflush(stdout);
      _exit(::testing::internal::skipped() ? 77 : (::testing::internal::failure_count() ? 1 : 0));
    }
    int status = 0;
    waitpid(pid, &status, 0);
    const char* verdict = "CRASH";
    if (WIFEXITED(status)) {
      int rc = WEXITSTATUS(status);
      verdict = rc == 0 ? "OK" : (rc == 77 ? "SKIP" : "FAIL");
    }
    if (std::strcmp(verdict, "OK") != 0 && std::strcmp(verdict, "SKIP") != 0) ++bad;
    std::printf("%s %s\n", verdict, full.c_str());
  }
  return bad ? 1 : 0;
}
