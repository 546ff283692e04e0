// Minimal stand-in for <gflags/gflags.h>: DEFINE_{string,bool,int32,uint32,int64,uint64,double},
// DECLARE_*, DEFINE_validator, ParseCommandLineFlags ("--name=value", "--name value", "--flag",
// "--noflag") and ShutDownCommandLineFlags.  Header-only; flag storage lives in the defining file.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <iostream>
#include <map>
#include <string>

namespace gflags {
struct FlagInfo {
    std::string type;
    void* ptr = nullptr;
    std::function<bool(const char*)> validate;   // reads *ptr
};
inline std::map<std::string, FlagInfo>& Registry() {
    static std::map<std::string, FlagInfo> r;
    return r;
}
inline std::map<const void*, std::string>& NameOf() {
    static std::map<const void*, std::string> r;
    return r;
}
struct FlagRegisterer {
    FlagRegisterer(const char* name, const char* type, void* ptr) {
        Registry()[name] = FlagInfo{type, ptr, nullptr};
        NameOf()[ptr] = name;
    }
};
template <typename T, typename F> bool RegisterFlagValidator(const T* flag, F fn) {
    auto it = NameOf().find(static_cast<const void*>(flag));
    if (it == NameOf().end()) return false;
    const std::string name = it->second;
    Registry()[name].validate = [flag, fn](const char* n) { return static_cast<bool>(fn(n, *flag)); };
    return true;
}
inline bool SetFromString(FlagInfo& f, const std::string& v) {
    try {
        if (f.type == "string") *static_cast<std::string*>(f.ptr) = v;
        else if (f.type == "bool") {
            *static_cast<bool*>(f.ptr) = (v == "true" || v == "1" || v == "yes" || v == "t" || v == "y" || v.empty());
        } else if (f.type == "int32") *static_cast<int32_t*>(f.ptr) = static_cast<int32_t>(std::stoll(v));
        else if (f.type == "uint32") *static_cast<uint32_t*>(f.ptr) = static_cast<uint32_t>(std::stoull(v));
        else if (f.type == "int64") *static_cast<int64_t*>(f.ptr) = static_cast<int64_t>(std::stoll(v));
        else if (f.type == "uint64") *static_cast<uint64_t*>(f.ptr) = static_cast<uint64_t>(std::stoull(v));
        else if (f.type == "double") *static_cast<double*>(f.ptr) = std::stod(v);
        else return false;
    } catch (...) { return false; }
    return true;
}
inline uint32_t ParseCommandLineFlags(int* argc, char*** argv, bool remove_flags) {
    int out = 1;
    char** av = *argv;
    for (int i = 1; i < *argc; ++i) {
        std::string a = av[i];
        if (a.rfind("--", 0) != 0 && a.rfind("-", 0) != 0) { av[out++] = av[i]; continue; }
        if (a == "--") { for (++i; i < *argc; ++i) av[out++] = av[i]; break; }
        std::string body = a.substr(a.rfind("--", 0) == 0 ? 2 : 1), name = body, value;
        bool has_value = false;
        const auto eq = body.find('=');
        if (eq != std::string::npos) { name = body.substr(0, eq); value = body.substr(eq + 1); has_value = true; }
        auto it = Registry().find(name);
        if (it == Registry().end() && name.rfind("no", 0) == 0) {
            auto it2 = Registry().find(name.substr(2));
            if (it2 != Registry().end() && it2->second.type == "bool") { *static_cast<bool*>(it2->second.ptr) = false; continue; }
        }
        if (it == Registry().end()) { std::cerr << "ERROR: unknown command line flag '" << name << "'\n"; std::exit(1); }
        if (!has_value) {
            if (it->second.type == "bool") value = "true";
            else if (i + 1 < *argc) value = av[++i];
            else { std::cerr << "ERROR: flag '--" << name << "' is missing its argument\n"; std::exit(1); }
        }
        if (!SetFromString(it->second, value)) {
            std::cerr << "ERROR: illegal value '" << value << "' specified for " << it->second.type << " flag '" << name << "'\n";
            std::exit(1);
        }
    }
    for (auto& kv : Registry())
        if (kv.second.validate && !kv.second.validate(kv.first.c_str())) {
            std::cerr << "ERROR: failed validation of new value for flag '" << kv.first << "'\n";
            std::exit(1);
        }
    if (remove_flags) { *argc = out; av[out] = nullptr; }
    return static_cast<uint32_t>(out);
}
inline void ShutDownCommandLineFlags() {}
}  // namespace gflags

#define ITB_DEFINE_FLAG(ctype, tname, name, dflt) \
    ctype FLAGS_##name = dflt;                    \
    static ::gflags::FlagRegisterer itb_flag_reg_##name(#name, tname, &FLAGS_##name)
#define DEFINE_string(name, dflt, help) ITB_DEFINE_FLAG(std::string, "string", name, dflt)
#define DEFINE_bool(name, dflt, help) ITB_DEFINE_FLAG(bool, "bool", name, dflt)
#define DEFINE_int32(name, dflt, help) ITB_DEFINE_FLAG(int32_t, "int32", name, dflt)
#define DEFINE_uint32(name, dflt, help) ITB_DEFINE_FLAG(uint32_t, "uint32", name, dflt)
#define DEFINE_int64(name, dflt, help) ITB_DEFINE_FLAG(int64_t, "int64", name, dflt)
#define DEFINE_uint64(name, dflt, help) ITB_DEFINE_FLAG(uint64_t, "uint64", name, dflt)
#define DEFINE_double(name, dflt, help) ITB_DEFINE_FLAG(double, "double", name, dflt)
#define DECLARE_string(name) extern std::string FLAGS_##name
#define DECLARE_bool(name) extern bool FLAGS_##name
#define DECLARE_int32(name) extern int32_t FLAGS_##name
#define DECLARE_uint32(name) extern uint32_t FLAGS_##name
#define DECLARE_int64(name) extern int64_t FLAGS_##name
#define DECLARE_uint64(name) extern uint64_t FLAGS_##name
#define DECLARE_double(name) extern double FLAGS_##name
#define DEFINE_validator(name, validator) \
    static const bool itb_flag_validator_##name = ::gflags::RegisterFlagValidator(&FLAGS_##name, validator)
