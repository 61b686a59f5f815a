// mstar-server: the native HTTP frontend as a stand-alone binary.
//   mstar-server --prefix <mesh prefix> [--host 0.0.0.0] [--port 8000] [--max-connections 1024]
// The Python API process (mstar_b200.api_server.native_frontend) starts it and answers on the "api_bridge" mailbox.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

extern "C" int mstar_http_serve(const char* prefix, const char* host, int port, int max_connections);

int main(int argc, char** argv) {
    std::string prefix = "mstar", host = "0.0.0.0";
    int port = 8000, maxc = 1024;
    for (int i = 1; i < argc; ++i) {
        auto next = [&](const char* name) -> const char* {
            if (i + 1 >= argc) { fprintf(stderr, "%s needs a value\n", name); exit(64); }
            return argv[++i];
        };
        if (!strcmp(argv[i], "--prefix")) prefix = next("--prefix");
        else if (!strcmp(argv[i], "--host")) host = next("--host");
        else if (!strcmp(argv[i], "--port")) port = atoi(next("--port"));
        else if (!strcmp(argv[i], "--max-connections")) maxc = atoi(next("--max-connections"));
        else if (!strcmp(argv[i], "--help")) {
            printf("usage: mstar-server --prefix P [--host H] [--port N] [--max-connections N]\n");
            return 0;
        } else { fprintf(stderr, "unknown argument %s\n", argv[i]); return 64; }
    }
    return mstar_http_serve(prefix.c_str(), host.c_str(), port, maxc);
}
