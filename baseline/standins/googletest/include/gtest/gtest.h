// Stand-in for the googletest 1.11 features the reference's test binary uses (TEST, EXPECT_EQ /
// EXPECT_TRUE / EXPECT_FALSE / EXPECT_FLOAT_EQ, a global Environment, InitGoogleTest, RUN_ALL_TESTS),
// so that the reference's own unit tests can run against the offline stand-ins.  Header only.
#pragma once

#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <iostream>
#include <string>
#include <vector>

namespace testing {

class Environment {
public:
  virtual ~Environment() {}
  virtual void SetUp() {}
  virtual void TearDown() {}
};

namespace internal {
struct Case {
  std::string name;
  std::function<void()> body;
};
inline std::vector<Case>& cases() {
  static std::vector<Case> c;
  return c;
}
inline std::vector<Environment*>& envs() {
  static std::vector<Environment*> e;
  return e;
}
inline int& failures() {
  static int f = 0;
  return f;
}
inline std::string& filter() {
  static std::string f;
  return f;
}
struct Registrar {
  Registrar(const char* suite, const char* name, std::function<void()> body) {
    cases().push_back({std::string(suite) + "." + name, std::move(body)});
  }
};
// Collects the text streamed after a failed check and prints it when the statement ends.
struct Reporter {
  bool failed;
  Reporter(bool f, const char* file, int line, const char* expr) : failed(f) {
    if (failed) {
      ++failures();
      std::cerr << file << ":" << line << ": Failure\n  " << expr << "\n";
    }
  }
  ~Reporter() {
    if (failed) std::cerr << std::endl;
  }
  template <typename T>
  Reporter& operator<<(const T& v) {
    if (failed) std::cerr << v;
    return *this;
  }
};
template <typename A, typename B>
bool Equal(const A& a, const B& b) {
  return a == b;
}
inline bool FloatEq(float a, float b) {
  if (std::isnan(a) || std::isnan(b)) return false;
  if (a == b) return true;
  int32_t ia, ib;
  std::memcpy(&ia, &a, 4);
  std::memcpy(&ib, &b, 4);
  if ((ia < 0) != (ib < 0)) return false;
  const int64_t d = static_cast<int64_t>(ia) - ib;
  return (d < 0 ? -d : d) <= 4;  // within 4 units in the last place, as googletest defines it
}
}  // namespace internal

inline Environment* AddGlobalTestEnvironment(Environment* env) {
  internal::envs().push_back(env);
  return env;
}

inline void InitGoogleTest(int* argc, char** argv) {
  for (int i = 1; i < *argc; ++i) {
    const std::string a = argv[i];
    const std::string key = "--gtest_filter=";
    if (a.compare(0, key.size(), key) == 0) internal::filter() = a.substr(key.size());
  }
}

}  // namespace testing

inline int RUN_ALL_TESTS() {
  using namespace testing::internal;
  for (auto* e : envs()) e->SetUp();
  int ran = 0, failed_cases = 0;
  for (auto& c : cases()) {
    if (!filter().empty() && filter() != "*") {
      std::string f = filter();
      if (!f.empty() && f.back() == '*') f.pop_back();
      if (c.name.compare(0, f.size(), f) != 0) continue;
    }
    const int before = failures();
    std::cout << "[ RUN      ] " << c.name << std::endl;
    c.body();
    ++ran;
    if (failures() != before) {
      ++failed_cases;
      std::cout << "[  FAILED  ] " << c.name << std::endl;
    } else {
      std::cout << "[       OK ] " << c.name << std::endl;
    }
  }
  for (auto it = envs().rbegin(); it != envs().rend(); ++it) (*it)->TearDown();
  std::cout << "[==========] " << ran << " tests ran, " << failed_cases << " failed." << std::endl;
  return failed_cases == 0 ? 0 : 1;
}

#define TEST(suite, name)                                                                            \
  static void kraken_gtest_##suite##_##name();                                                       \
  static ::testing::internal::Registrar kraken_gtest_reg_##suite##_##name(#suite, #name,             \
                                                                          kraken_gtest_##suite##_##name); \
  static void kraken_gtest_##suite##_##name()

#define EXPECT_TRUE(cond) ::testing::internal::Reporter(!(cond), __FILE__, __LINE__, "EXPECT_TRUE(" #cond ")")
#define EXPECT_FALSE(cond) ::testing::internal::Reporter(!!(cond), __FILE__, __LINE__, "EXPECT_FALSE(" #cond ")")
#define EXPECT_EQ(a, b) \
  ::testing::internal::Reporter(!::testing::internal::Equal((a), (b)), __FILE__, __LINE__, "EXPECT_EQ(" #a ", " #b ")")
#define EXPECT_FLOAT_EQ(a, b) \
  ::testing::internal::Reporter(!::testing::internal::FloatEq((a), (b)), __FILE__, __LINE__, "EXPECT_FLOAT_EQ(" #a ", " #b ")")
