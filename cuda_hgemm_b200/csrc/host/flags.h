// A small stand-in for gflags, which the reference depends on (src/main.cu:7,35-45,48) but
// which is a separate library. It accepts the reference's command lines unchanged:
// -flag=value, --flag=value, -flag value, and bare -boolflag / -noboolflag.
// Written for this driver; only the DEFINE_* / FLAGS_* / ParseCommandLineFlags names are shared.
#pragma once

#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

namespace flags {

enum class Kind { kBool, kUint32, kUint64, kDouble, kString };

struct Entry {
    const char *name;
    Kind kind;
    void *storage;
    const char *help;
};

inline std::vector<Entry> &registry() {
    static std::vector<Entry> entries;
    return entries;
}

struct Registrar {
    Registrar(const char *name, Kind kind, void *storage, const char *help) {
        registry().push_back({name, kind, storage, help});
    }
};

inline bool parse_bool(const std::string &v, bool *out) {
    if (v == "true" || v == "1" || v == "yes" || v == "on" || v == "t" || v == "y") return *out = true, true;
    if (v == "false" || v == "0" || v == "no" || v == "off" || v == "f" || v == "n") return *out = false, true;
    return false;
}

inline bool assign(const Entry &e, const std::string &v) {
    char *end = nullptr;
    switch (e.kind) {
        case Kind::kBool: return parse_bool(v, static_cast<bool *>(e.storage));
        case Kind::kUint32: {
            if (v.empty() || v[0] == '-') return false;
            unsigned long long x = strtoull(v.c_str(), &end, 10);
            if (*end || x > 0xFFFFFFFFull) return false;
            *static_cast<uint32_t *>(e.storage) = static_cast<uint32_t>(x);
            return true;
        }
        case Kind::kUint64: {
            if (v.empty() || v[0] == '-') return false;
            *static_cast<uint64_t *>(e.storage) = strtoull(v.c_str(), &end, 10);
            return *end == 0;
        }
        case Kind::kDouble:
            *static_cast<double *>(e.storage) = strtod(v.c_str(), &end);
            return !v.empty() && *end == 0;
        case Kind::kString: *static_cast<std::string *>(e.storage) = v; return true;
    }
    return false;
}

inline void usage(const char *prog) {
    fprintf(stderr, "usage: %s [-flag=value ...]\n", prog);
    for (const Entry &e : registry()) fprintf(stderr, "  -%s  %s\n", e.name, e.help);
}

// Returns the index of the first non-flag argument. Unknown flags and bad values end the process
// with status 1, as gflags does.
inline int ParseCommandLineFlags(int *argc, char ***argv, bool /*remove_flags*/) {
    int i = 1;
    for (; i < *argc; ++i) {
        std::string arg = (*argv)[i];
        if (arg == "--") {
            ++i;
            break;
        }
        if (arg.size() < 2 || arg[0] != '-') break;
        arg = arg.substr(arg[1] == '-' ? 2 : 1);
        if (arg == "help" || arg == "h") {
            usage((*argv)[0]);
            exit(0);
        }
        std::string name = arg, value;
        bool has_value = false;
        const size_t eq = arg.find('=');
        if (eq != std::string::npos) {
            name = arg.substr(0, eq);
            value = arg.substr(eq + 1);
            has_value = true;
        }
        const Entry *found = nullptr;
        bool negated = false;
        for (const Entry &e : registry()) {
            if (name == e.name) found = &e;
        }
        if (!found && name.compare(0, 2, "no") == 0) {
            for (const Entry &e : registry()) {
                if (e.kind == Kind::kBool && name.substr(2) == e.name) found = &e, negated = true;
            }
        }
        if (!found) {
            fprintf(stderr, "ERROR: unknown command line flag '%s'\n", name.c_str());
            exit(1);
        }
        if (!has_value) {
            if (found->kind == Kind::kBool) {
                value = negated ? "false" : "true";
            } else if (i + 1 < *argc) {
                value = (*argv)[++i];
            } else {
                fprintf(stderr, "ERROR: flag '%s' is missing its argument\n", name.c_str());
                exit(1);
            }
        }
        if (!assign(*found, value)) {
            fprintf(stderr, "ERROR: illegal value '%s' specified for flag '%s'\n", value.c_str(), name.c_str());
            exit(1);
        }
    }
    return i;
}

inline void ShutDownCommandLineFlags() {}

}  // namespace flags

#define GFLAGS_NAMESPACE flags

#define HGEMM_DEFINE_FLAG(type, kind, name, value, help) \
    type FLAGS_##name = value;                           \
    static ::flags::Registrar flag_registrar_##name(#name, ::flags::Kind::kind, &FLAGS_##name, help)

#define DEFINE_bool(name, value, help) HGEMM_DEFINE_FLAG(bool, kBool, name, value, help)
#define DEFINE_uint32(name, value, help) HGEMM_DEFINE_FLAG(uint32_t, kUint32, name, value, help)
#define DEFINE_uint64(name, value, help) HGEMM_DEFINE_FLAG(uint64_t, kUint64, name, value, help)
#define DEFINE_double(name, value, help) HGEMM_DEFINE_FLAG(double, kDouble, name, value, help)
#define DEFINE_string(name, value, help) HGEMM_DEFINE_FLAG(std::string, kString, name, value, help)
