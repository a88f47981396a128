/*
 * uccl_selftest.h -- native unit tests compiled into the library.
 *
 * The host runtime is C++; its unit tests are C++ too and are reachable through these three
 * entry points so that pytest (or any other driver) can run them one by one without a GPU.
 */
#ifndef UCCL_SELFTEST_H_
#define UCCL_SELFTEST_H_
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

int ucclSelfTestCount(void);
const char* ucclSelfTestName(int index);
/* Returns 0 on success; `report` receives a human-readable log (always NUL terminated). */
int ucclSelfTestRun(const char* name, char* report, size_t reportLen);

#ifdef __cplusplus
}
#endif
#endif
