// Native HTTP/1.1 frontend. The binary `mstar-server` accepts client connections, parses requests and streams
// responses; the Python API process keeps media loading, prompt processing and the conductor protocol. The two talk
// over the shared-memory control mesh (entities "frontend" and "api_bridge"):
//
//   frontend -> api_bridge :  {"id":N,"method":"POST","path":"/generate","query":"..","content_type":"..","len":L}\n<body>
//   api_bridge -> frontend :  {"id":N,"kind":"head","status":200,"content_type":"..","streaming":true}\n
//                             {"id":N,"kind":"chunk"}\n<bytes>            (any number)
//                             {"kind":"b64_batch","n":K}\n<K records>     body chunks of K requests in one message:
//                               record = u64 id, u32 prefix_len, u32 data_len, u32 suffix_len (little endian), then the
//                               three byte strings; the chunk is prefix + base64(data) + suffix (an NDJSON line whose
//                               binary field is encoded here instead of in the API process)
//                             {"id":N,"kind":"end"}\n
//
// Streaming responses go out with chunked transfer encoding as the chunks arrive; other responses are buffered and
// sent with a Content-Length. One thread per connection (bounded), one thread draining the mailbox and handing
// frames to the waiting connection threads. /health and /frontend_stats are answered here without a round trip.
//
// Reference counterpart: the Rust `mstar-server` frontend (rust/server/, selected with --rust-frontend in
// mstar/api_server/entrypoint.py:888-905), which bridges to the Python process through a socket directory.
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <sys/socket.h>
#include <unistd.h>

extern "C" {
void* mstar_mesh_create(const char* prefix, const char* entity, unsigned long long ring_bytes);
int mstar_mesh_send(void* handle, const char* dst, const char* payload, unsigned long long len);
long long mstar_mesh_recv(void* handle, char* out, unsigned long long cap, int timeout_ms);
long long mstar_mesh_peek_size(void* handle);
void mstar_mesh_destroy(void* handle, int unlink_own);
}

namespace {

struct Frame {
    std::string kind;          // head | chunk | end
    int status = 200;
    std::string content_type;
    bool streaming = false;
    std::string payload;
};

struct Pending {
    std::mutex m;
    std::condition_variable cv;
    std::deque<Frame> frames;
};

struct Server {
    void* mesh = nullptr;
    std::mutex send_m;
    std::mutex map_m;
    std::map<uint64_t, std::shared_ptr<Pending>> pending;
    std::atomic<uint64_t> next_id{1};
    std::atomic<bool> running{true};
    std::atomic<bool> bridge_ready{false};
    std::atomic<int> active{0};
    std::atomic<uint64_t> served{0}, errors{0}, bytes_in{0}, bytes_out{0};
    int max_connections = 1024;
    size_t max_body = 1ull << 30;
    int request_timeout_ms = 600000;
};

// ---- tiny JSON helpers for the one-line headers (flat objects, string / number / bool values) ----
std::string json_escape(const std::string& s) {
    std::string o;
    for (unsigned char c : s) {
        if (c == '"' || c == '\\') { o += '\\'; o += (char)c; }
        else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else o += (char)c;
    }
    return o;
}

bool json_get(const std::string& j, const std::string& key, std::string* out) {
    const std::string pat = "\"" + key + "\":";
    size_t p = j.find(pat);
    if (p == std::string::npos) return false;
    p += pat.size();
    while (p < j.size() && j[p] == ' ') ++p;
    if (p >= j.size()) return false;
    if (j[p] == '"') {
        std::string v;
        for (++p; p < j.size() && j[p] != '"'; ++p) {
            if (j[p] == '\\' && p + 1 < j.size()) ++p;
            v += j[p];
        }
        *out = v;
        return true;
    }
    size_t e = p;
    while (e < j.size() && j[e] != ',' && j[e] != '}') ++e;
    *out = j.substr(p, e - p);
    return true;
}

void base64_append(std::string& out, const unsigned char* p, size_t n) {
    static const char T[] = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
    size_t o = out.size();
    out.resize(o + (n + 2) / 3 * 4);
    char* w = &out[o];
    size_t i = 0;
    for (; i + 2 < n; i += 3) {
        const unsigned v = (p[i] << 16) | (p[i + 1] << 8) | p[i + 2];
        *w++ = T[v >> 18]; *w++ = T[(v >> 12) & 63]; *w++ = T[(v >> 6) & 63]; *w++ = T[v & 63];
    }
    if (i < n) {
        const unsigned v = (p[i] << 16) | (i + 1 < n ? p[i + 1] << 8 : 0);
        *w++ = T[v >> 18]; *w++ = T[(v >> 12) & 63];
        *w++ = i + 1 < n ? T[(v >> 6) & 63] : '=';
        *w++ = '=';
    }
}

bool send_all(int fd, const char* p, size_t n) {
    while (n) {
        ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
        if (w <= 0) return false;
        p += w;
        n -= (size_t)w;
    }
    return true;
}

bool send_str(int fd, const std::string& s) { return send_all(fd, s.data(), s.size()); }

const char* reason(int status) {
    switch (status) {
        case 200: return "OK";
        case 400: return "Bad Request";
        case 404: return "Not Found";
        case 413: return "Payload Too Large";
        case 422: return "Unprocessable Entity";
        case 500: return "Internal Server Error";
        case 503: return "Service Unavailable";
        case 504: return "Gateway Timeout";
        default: return "Status";
    }
}

void simple_response(Server* S, int fd, int status, const std::string& ctype, const std::string& body) {
    char head[512];
    int n = snprintf(head, sizeof head,
                     "HTTP/1.1 %d %s\r\nContent-Type: %s\r\nContent-Length: %zu\r\nConnection: close\r\n\r\n", status,
                     reason(status), ctype.c_str(), body.size());
    send_all(fd, head, (size_t)n);
    send_str(fd, body);
    S->bytes_out += body.size();
}

std::string lower(std::string s) {
    for (auto& c : s) c = (char)tolower((unsigned char)c);
    return s;
}

// Reads one request: returns false on a malformed / oversized request (a response has been written).
bool read_request(Server* S, int fd, std::string* method, std::string* target, std::string* ctype, std::string* body) {
    std::string buf;
    char tmp[16384];
    size_t hdr_end = std::string::npos;
    while (hdr_end == std::string::npos) {
        ssize_t r = ::recv(fd, tmp, sizeof tmp, 0);
        if (r <= 0) return false;
        buf.append(tmp, (size_t)r);
        hdr_end = buf.find("\r\n\r\n");
        if (buf.size() > (1u << 20) && hdr_end == std::string::npos) {
            simple_response(S, fd, 400, "text/plain", "header too large");
            return false;
        }
    }
    const std::string head = buf.substr(0, hdr_end);
    size_t le = head.find("\r\n");
    const std::string line = head.substr(0, le);
    size_t s1 = line.find(' '), s2 = line.rfind(' ');
    if (s1 == std::string::npos || s2 == s1) {
        simple_response(S, fd, 400, "text/plain", "bad request line");
        return false;
    }
    *method = line.substr(0, s1);
    *target = line.substr(s1 + 1, s2 - s1 - 1);
    size_t clen = 0;
    bool expect_continue = false;
    size_t p = le == std::string::npos ? head.size() : le + 2;
    while (p < head.size()) {
        size_t e = head.find("\r\n", p);
        if (e == std::string::npos) e = head.size();
        const std::string h = head.substr(p, e - p);
        size_t c = h.find(':');
        if (c != std::string::npos) {
            const std::string k = lower(h.substr(0, c));
            std::string v = h.substr(c + 1);
            while (!v.empty() && v[0] == ' ') v.erase(0, 1);
            if (k == "content-length") clen = (size_t)strtoull(v.c_str(), nullptr, 10);
            else if (k == "content-type") *ctype = v;
            else if (k == "expect" && lower(v) == "100-continue") expect_continue = true;
        }
        p = e + 2;
    }
    if (clen > S->max_body) {
        simple_response(S, fd, 413, "text/plain", "body too large");
        return false;
    }
    if (expect_continue) send_str(fd, "HTTP/1.1 100 Continue\r\n\r\n");
    *body = buf.substr(hdr_end + 4);
    while (body->size() < clen) {
        ssize_t r = ::recv(fd, tmp, sizeof tmp, 0);
        if (r <= 0) return false;
        body->append(tmp, (size_t)r);
    }
    body->resize(clen);
    S->bytes_in += clen;
    return true;
}

void handle_connection(Server* S, int fd) {
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
    std::string method, target, ctype, body;
    if (!read_request(S, fd, &method, &target, &ctype, &body)) {
        ::close(fd);
        S->active--;
        return;
    }
    std::string path = target, query;
    size_t q = target.find('?');
    if (q != std::string::npos) { path = target.substr(0, q); query = target.substr(q + 1); }
    if (path == "/frontend_stats") {
        char b[256];
        snprintf(b, sizeof b, "{\"served\":%llu,\"errors\":%llu,\"active\":%d,\"bytes_in\":%llu,\"bytes_out\":%llu}",
                 (unsigned long long)S->served.load(), (unsigned long long)S->errors.load(), S->active.load(),
                 (unsigned long long)S->bytes_in.load(), (unsigned long long)S->bytes_out.load());
        simple_response(S, fd, 200, "application/json", b);
    } else if (path == "/health" && !S->bridge_ready.load()) {
        simple_response(S, fd, 503, "application/json", "{\"status\":\"starting\"}");
    } else {
        const uint64_t id = S->next_id++;
        auto pend = std::make_shared<Pending>();
        {
            std::lock_guard<std::mutex> g(S->map_m);
            S->pending[id] = pend;
        }
        std::string msg = "{\"id\":" + std::to_string(id) + ",\"method\":\"" + json_escape(method) + "\",\"path\":\"" +
                          json_escape(path) + "\",\"query\":\"" + json_escape(query) + "\",\"content_type\":\"" +
                          json_escape(ctype) + "\",\"len\":" + std::to_string(body.size()) + "}\n";
        msg += body;
        int rc;
        {
            std::lock_guard<std::mutex> g(S->send_m);
            rc = mstar_mesh_send(S->mesh, "api_bridge", msg.data(), msg.size());
        }
        if (rc != 0) {
            simple_response(S, fd, 503, "application/json", "{\"detail\":\"API process is not reachable\"}");
            S->errors++;
        } else {
            bool head_sent = false, streaming = false, done = false, client_ok = true;
            std::string buffered, buffered_type = "application/json";
            int status = 200;
            while (!done) {
                Frame f;
                {
                    std::unique_lock<std::mutex> lk(pend->m);
                    if (!pend->cv.wait_for(lk, std::chrono::milliseconds(S->request_timeout_ms),
                                           [&] { return !pend->frames.empty() || !S->running.load(); })) {
                        f.kind = "timeout";
                    } else if (pend->frames.empty()) {
                        f.kind = "timeout";
                    } else {
                        f = std::move(pend->frames.front());
                        pend->frames.pop_front();
                    }
                }
                if (f.kind == "head") {
                    status = f.status;
                    streaming = f.streaming;
                    buffered_type = f.content_type.empty() ? "application/json" : f.content_type;
                    if (streaming) {
                        char h[512];
                        int n = snprintf(h, sizeof h,
                                         "HTTP/1.1 %d %s\r\nContent-Type: %s\r\nTransfer-Encoding: chunked\r\n"
                                         "Cache-Control: no-cache\r\nConnection: close\r\n\r\n",
                                         status, reason(status), buffered_type.c_str());
                        client_ok = send_all(fd, h, (size_t)n);
                        head_sent = true;
                    }
                } else if (f.kind == "chunk") {
                    if (streaming) {
                        if (client_ok && !f.payload.empty()) {
                            char sz[32];
                            int n = snprintf(sz, sizeof sz, "%zx\r\n", f.payload.size());
                            client_ok = send_all(fd, sz, (size_t)n) && send_str(fd, f.payload) && send_str(fd, "\r\n");
                            S->bytes_out += f.payload.size();
                        }
                    } else {
                        buffered += f.payload;
                    }
                } else if (f.kind == "end") {
                    if (streaming) {
                        if (client_ok) send_str(fd, "0\r\n\r\n");
                    } else {
                        simple_response(S, fd, status, buffered_type, buffered);
                    }
                    done = true;
                } else {       // timeout or shutdown
                    if (!head_sent) simple_response(S, fd, 504, "application/json", "{\"detail\":\"timed out\"}");
                    S->errors++;
                    done = true;
                }
                if (!client_ok && streaming && !done) {
                    // the client went away: tell the API process so that it can abort the request, then stop
                    std::string ab = "{\"id\":" + std::to_string(id) + ",\"method\":\"ABORT\",\"path\":\"\",\"query\":\"\","
                                     "\"content_type\":\"\",\"len\":0}\n";
                    std::lock_guard<std::mutex> g(S->send_m);
                    mstar_mesh_send(S->mesh, "api_bridge", ab.data(), ab.size());
                    done = true;
                }
            }
        }
        std::lock_guard<std::mutex> g(S->map_m);
        S->pending.erase(id);
    }
    S->served++;
    ::shutdown(fd, SHUT_RDWR);
    ::close(fd);
    S->active--;
}

void mailbox_loop(Server* S) {
    std::vector<char> buf(1 << 20);
    while (S->running.load()) {
        long long n = mstar_mesh_recv(S->mesh, buf.data(), buf.size(), 100);
        if (n == -3) {
            long long need = mstar_mesh_peek_size(S->mesh);
            buf.resize((size_t)std::max<long long>(need, (long long)buf.size() * 2));
            n = mstar_mesh_recv(S->mesh, buf.data(), buf.size(), 0);
        }
        if (n <= 0) continue;
        const char* nl = (const char*)memchr(buf.data(), '\n', (size_t)n);
        if (!nl) continue;
        const std::string hdr(buf.data(), nl - buf.data());
        std::string v;
        if (json_get(hdr, "kind", &v) && v == "ready") {
            S->bridge_ready = true;
            continue;
        }
        if (v == "shutdown") {
            S->running = false;
            break;
        }
        if (v == "b64_batch") {
            const unsigned char* q = (const unsigned char*)nl + 1;
            const unsigned char* end = (const unsigned char*)buf.data() + n;
            while ((size_t)(end - q) >= 20) {
                uint64_t id;
                uint32_t lens[3];
                memcpy(&id, q, 8);
                memcpy(lens, q + 8, 12);
                q += 20;
                if ((uint64_t)lens[0] + lens[1] + lens[2] > (uint64_t)(end - q)) break;       // malformed: drop the rest
                Frame f;
                f.kind = "chunk";
                f.payload.reserve(lens[0] + (lens[1] + 2) / 3 * 4 + lens[2]);
                f.payload.assign((const char*)q, lens[0]);
                base64_append(f.payload, q + lens[0], lens[1]);
                f.payload.append((const char*)q + lens[0] + lens[1], lens[2]);
                q += (size_t)lens[0] + lens[1] + lens[2];
                std::shared_ptr<Pending> p;
                {
                    std::lock_guard<std::mutex> g(S->map_m);
                    auto it = S->pending.find(id);
                    if (it != S->pending.end()) p = it->second;
                }
                if (!p) continue;
                {
                    std::lock_guard<std::mutex> g(p->m);
                    p->frames.push_back(std::move(f));
                }
                p->cv.notify_one();
            }
            continue;
        }
        Frame f;
        f.kind = v;
        uint64_t id = 0;
        if (json_get(hdr, "id", &v)) id = strtoull(v.c_str(), nullptr, 10);
        if (json_get(hdr, "status", &v)) f.status = atoi(v.c_str());
        if (json_get(hdr, "content_type", &v)) f.content_type = v;
        if (json_get(hdr, "streaming", &v)) f.streaming = (v == "true");
        f.payload.assign(nl + 1, (size_t)n - (size_t)(nl + 1 - buf.data()));
        std::shared_ptr<Pending> p;
        {
            std::lock_guard<std::mutex> g(S->map_m);
            auto it = S->pending.find(id);
            if (it != S->pending.end()) p = it->second;
        }
        if (!p) continue;      // the connection is gone
        {
            std::lock_guard<std::mutex> g(p->m);
            p->frames.push_back(std::move(f));
        }
        p->cv.notify_one();
    }
}

}  // namespace

// Runs until a shutdown frame arrives or the process is signalled. Returns 0 on a clean exit.
extern "C" __attribute__((visibility("default"))) int mstar_http_serve(const char* prefix, const char* host, int port,
                                                                        int max_connections) {
    signal(SIGPIPE, SIG_IGN);
    Server S;
    S.max_connections = max_connections > 0 ? max_connections : 1024;
    S.mesh = mstar_mesh_create(prefix, "frontend", 64ull << 20);
    if (!S.mesh) {
        fprintf(stderr, "mstar-server: cannot create the mailbox %s/frontend\n", prefix);
        return 2;
    }
    int ls = ::socket(AF_INET, SOCK_STREAM, 0);
    int one = 1;
    setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, host, &addr.sin_addr) != 1) addr.sin_addr.s_addr = htonl(INADDR_ANY);
    if (::bind(ls, (sockaddr*)&addr, sizeof addr) != 0 || ::listen(ls, 1024) != 0) {
        perror("mstar-server: bind/listen");
        return 3;
    }
    timeval tv{0, 200000};
    setsockopt(ls, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
    std::thread mb(mailbox_loop, &S);
    fprintf(stderr, "mstar-server: listening on %s:%d\n", host, port);
    while (S.running.load()) {
        int fd = ::accept(ls, nullptr, nullptr);
        if (fd < 0) continue;
        if (S.active.load() >= S.max_connections) {
            simple_response(&S, fd, 503, "application/json", "{\"detail\":\"too many connections\"}");
            ::close(fd);
            continue;
        }
        S.active++;
        std::thread(handle_connection, &S, fd).detach();
    }
    ::close(ls);
    mb.join();
    for (int i = 0; i < 100 && S.active.load() > 0; ++i) usleep(20000);
    mstar_mesh_destroy(S.mesh, 1);
    return 0;
}
