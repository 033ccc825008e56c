/* Stand-in for the part of gflags the reference's partitioner uses (EBV_mpi.cpp:9-18,119): DEFINE_string / _bool /
 * _uint64 / _double and google::ParseCommandLineFlags.  Accepts -name value, --name value, -name=value, --name=value;
 * a bool flag may stand alone (-is_dump) or carry =true / =false.  Unknown flags end the program.
 * Test infrastructure for oracle/_ref only. */
#ifndef DRONE_ORACLE_EBV_GFLAGS_STANDIN_H
#define DRONE_ORACLE_EBV_GFLAGS_STANDIN_H
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace gflags_standin {

struct Flag {
    const char *name;
    char kind;     /* 's' string, 'b' bool, 'u' uint64, 'd' double */
    void *value;
};

inline std::vector<Flag> &registry() {
    static std::vector<Flag> flags;
    return flags;
}

struct Registrar {
    Registrar(const char *name, char kind, void *value) { registry().push_back({name, kind, value}); }
};

inline void assign(const Flag &f, const char *text) {
    switch (f.kind) {
    case 's': *static_cast<std::string *>(f.value) = text; break;
    case 'b': *static_cast<bool *>(f.value) = !(std::strcmp(text, "false") == 0 || std::strcmp(text, "0") == 0); break;
    case 'u': *static_cast<uint64_t *>(f.value) = std::strtoull(text, nullptr, 10); break;
    case 'd': *static_cast<double *>(f.value) = std::strtod(text, nullptr); break;
    }
}

}  // namespace gflags_standin

#define DEFINE_string(name, dflt, help)                                                                              \
    std::string FLAGS_##name = dflt;                                                                                 \
    static gflags_standin::Registrar flag_registrar_##name(#name, 's', &FLAGS_##name)
#define DEFINE_bool(name, dflt, help)                                                                                \
    bool FLAGS_##name = dflt;                                                                                        \
    static gflags_standin::Registrar flag_registrar_##name(#name, 'b', &FLAGS_##name)
#define DEFINE_uint64(name, dflt, help)                                                                              \
    uint64_t FLAGS_##name = dflt;                                                                                    \
    static gflags_standin::Registrar flag_registrar_##name(#name, 'u', &FLAGS_##name)
#define DEFINE_double(name, dflt, help)                                                                              \
    double FLAGS_##name = dflt;                                                                                      \
    static gflags_standin::Registrar flag_registrar_##name(#name, 'd', &FLAGS_##name)

namespace google {

inline unsigned ParseCommandLineFlags(int *argc, char ***argv, bool) {
    using namespace gflags_standin;
    int i = 1;
    for (; i < *argc; ++i) {
        const char *arg = (*argv)[i];
        if (arg[0] != '-') break;
        const char *body = arg + (arg[1] == '-' ? 2 : 1);
        const char *eq = std::strchr(body, '=');
        const std::string name = eq ? std::string(body, eq) : std::string(body);
        const Flag *flag = nullptr;
        for (const Flag &f : registry())
            if (name == f.name) flag = &f;
        if (!flag) {
            std::fprintf(stderr, "unknown flag %s\n", arg);
            std::exit(2);
        }
        if (eq) {
            assign(*flag, eq + 1);
        } else if (flag->kind == 'b') {
            *static_cast<bool *>(flag->value) = true;
        } else {
            if (i + 1 >= *argc) {
                std::fprintf(stderr, "flag %s needs a value\n", arg);
                std::exit(2);
            }
            assign(*flag, (*argv)[++i]);
        }
    }
    return (unsigned)i;
}

}  // namespace google
#endif
