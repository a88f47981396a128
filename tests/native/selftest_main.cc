// Runs the library's native self tests from a plain executable, so that they can be built with
// -fsanitize=address,undefined or -fsanitize=thread (`make asan`, `make tsan`): the host runtime's
// race and memory-error check, in place of device-side sanitizers.
#include <stdio.h>
#include <string.h>

#include "uccl_selftest.h"

int main(int argc, char** argv) {
  int failed = 0;
  static char report[1 << 16];
  for (int i = 0; i < ucclSelfTestCount(); ++i) {
    const char* name = ucclSelfTestName(i);
    if (argc > 1 && strcmp(argv[1], name) != 0) continue;
    const int rc = ucclSelfTestRun(name, report, sizeof(report));
    printf("%-28s %s\n", name, rc == 0 ? "ok" : "FAILED");
    if (rc != 0) {
      printf("%s\n", report);
      ++failed;
    }
  }
  return failed ? 1 : 0;
}
