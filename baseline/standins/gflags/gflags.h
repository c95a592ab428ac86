// Stand-in for the gflags 2.2 macros and calls used by the reference's two main() files
// (kraken/executable/ps_server_main.cc:5-14, scheduler_server_main.cc:5-9): DEFINE_uint32 /
// DEFINE_string registering FLAGS_<name>, and ParseCommandLineFlags accepting --name=value,
// --name value and the single-dash forms.  Header only, for the offline baseline build.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <map>
#include <string>

namespace gflags {

struct Registry {
  static std::map<std::string, std::function<bool(const char*)>>& setters() {
    static std::map<std::string, std::function<bool(const char*)>> m;
    return m;
  }
  static std::string& usage() {
    static std::string u;
    return u;
  }
};

struct Registrar {
  Registrar(const char* name, std::function<bool(const char*)> set) { Registry::setters()[name] = std::move(set); }
};

inline void SetUsageMessage(const std::string& u) { Registry::usage() = u; }

inline uint32_t ParseCommandLineFlags(int* argc, char*** argv, bool /*remove_flags*/) {
  int i = 1;
  for (; i < *argc; ++i) {
    const char* a = (*argv)[i];
    if (a[0] != '-') break;
    while (*a == '-') ++a;
    std::string name(a), value;
    bool has_value = false;
    const size_t eq = name.find('=');
    if (eq != std::string::npos) {
      value = name.substr(eq + 1);
      name = name.substr(0, eq);
      has_value = true;
    }
    auto it = Registry::setters().find(name);
    if (it == Registry::setters().end()) {
      std::fprintf(stderr, "unknown flag --%s\n%s\n", name.c_str(), Registry::usage().c_str());
      std::exit(1);
    }
    if (!has_value) {
      if (i + 1 >= *argc) {
        std::fprintf(stderr, "flag --%s needs a value\n", name.c_str());
        std::exit(1);
      }
      value = (*argv)[++i];
    }
    if (!it->second(value.c_str())) {
      std::fprintf(stderr, "bad value '%s' for flag --%s\n", value.c_str(), name.c_str());
      std::exit(1);
    }
  }
  return static_cast<uint32_t>(i);
}

}  // namespace gflags

#define KRAKEN_BASELINE_DEFINE_NUM(type, name, def, parse)                                   \
  type FLAGS_##name = (def);                                                                 \
  static ::gflags::Registrar kraken_flag_registrar_##name(#name, [](const char* v) -> bool { \
    char* end = nullptr;                                                                     \
    FLAGS_##name = static_cast<type>(parse(v, &end, 10));                                    \
    return end != v && *end == '\0';                                                         \
  })

#define DEFINE_uint32(name, def, help) KRAKEN_BASELINE_DEFINE_NUM(uint32_t, name, def, std::strtoul)
#define DEFINE_int32(name, def, help) KRAKEN_BASELINE_DEFINE_NUM(int32_t, name, def, std::strtol)
#define DEFINE_uint64(name, def, help) KRAKEN_BASELINE_DEFINE_NUM(uint64_t, name, def, std::strtoull)
#define DEFINE_int64(name, def, help) KRAKEN_BASELINE_DEFINE_NUM(int64_t, name, def, std::strtoll)

#define DEFINE_string(name, def, help)                                                       \
  std::string FLAGS_##name = (def);                                                          \
  static ::gflags::Registrar kraken_flag_registrar_##name(#name, [](const char* v) -> bool { \
    FLAGS_##name = v;                                                                        \
    return true;                                                                             \
  })
