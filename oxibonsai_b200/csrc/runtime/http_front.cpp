// Native HTTP/1.1 + server-sent-events front.
//
// The reference serves through axum / hyper (crates/oxibonsai-runtime/src/server.rs:203-243) and frames streamed tokens as
// SSE events "role chunk -> content chunks -> finish chunk -> [DONE]" with UTF-8-safe incremental decoding (:391-512).
// Here the sockets, the HTTP parsing and - for token streams - the whole per-token path (token id -> bytes, UTF-8
// boundary and stop-sequence hold-back, JSON escaping, SSE + chunked framing, the write) live in this file, behind a C
// ABI.  The Python side only sees whole requests (it answers them through the ASGI application) and, for a stream, calls
// bfront_stream_push(token) from the scheduler thread: no interpreter work per token beyond that call.
//
// Threads: one I/O thread (epoll) owns every socket, does every recv / send (without holding the mutex) and is the only
// one that removes connections.  Other threads append to a connection's output buffer under the front's mutex and wake the
// I/O thread through an eventfd; parsed requests and disconnect notices reach Python through a queue that
// bfront_next_event() blocks on.
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace bonsai_front {

constexpr size_t kMaxHeader = 64 * 1024;
constexpr size_t kMaxBody = 256u * 1024 * 1024;
constexpr size_t kMaxOut = 256u * 1024 * 1024;      // a client that reads nothing is dropped beyond this

using Clock = std::chrono::steady_clock;

enum ConnState { READING = 0, DISPATCHED = 1, RESPONDING = 2, STREAMING = 3 };
enum StreamState { LIVE = 0, STOP_HIT = 1, CLIENT_GONE = 2, TIMED_OUT = 3, FINISHED = 4 };

struct Conn {
    int fd = -1;
    int64_t id = 0;
    std::string in;                     // bytes received and not parsed yet (I/O thread only)
    std::string out;                    // bytes to send, appended by any thread under the front's mutex
    std::string wire;                   // bytes being sent (I/O thread only; refilled from ``out`` when empty)
    size_t wire_off = 0;
    bool reparse = false;               // a response was completed: look for a pipelined request in ``in``
    int state = READING;
    bool keep_alive = true;
    bool close_after_flush = false;
    bool want_write = false;            // EPOLLOUT registered
    bool continued = false;             // "100 Continue" already sent for the request being read
    bool head_only = false;             // the request being answered is a HEAD: headers as for GET, no body bytes
    bool http10 = false;                // the request came as HTTP/1.0: no chunked framing, the body ends with the connection
    Clock::time_point last_io = Clock::now();   // last byte received or sent (I/O thread only)
    int64_t stream = 0;
    std::string peer;
};

struct Stream {
    int64_t id = 0, conn = 0;
    std::string head;                   // fixed front part of every chunk's JSON
    bool chat = true;
    std::vector<std::string> stops;
    std::string first_event;            // the role chunk of a chat stream (may be empty)
    std::string held;                   // decoded bytes not sent yet: incomplete UTF-8 or a possible start of a stop sequence
    std::string early;                  // framed events produced before the response head was written
    bool begun = false;
    bool raw = false;                   // HTTP/1.0 client: events go out unframed and the connection is closed at the end
    int state = LIVE;
    Clock::time_point deadline;
    bool has_deadline = false;
    uint64_t tokens = 0, events = 0;
};

struct Event {                          // what Python receives
    int kind = 0;                       // 1 request, 2 connection closed
    int64_t conn = 0;
    std::string method, target, headers, body, peer;
};

struct Front {
    int listen_fd = -1, ep = -1, wake = -1, port = 0;
    std::string host;
    std::thread io;
    std::atomic<bool> stopping{false};
    std::atomic<bool> wake_pending{false};
    std::atomic<int> idle_timeout_ms{75000};   // a connection that waits for a request and moves no byte for this long is closed (0: never)
    std::atomic<bool> lazy{false};      // token pushes do not wake the I/O thread; the producer calls bfront_kick() once per step
    std::mutex mu;
    std::condition_variable cv;
    std::deque<Event> events;
    std::unordered_map<int64_t, std::unique_ptr<Conn>> conns;
    std::unordered_map<int64_t, std::unique_ptr<Stream>> streams;
    std::vector<int64_t> dirty;         // connections with new output (filled by other threads)
    int64_t next_id = 1;
    std::vector<uint8_t> vocab_bytes;
    std::vector<uint32_t> vocab_off;    // n + 1 offsets
    ~Front() {                        // process exit with the front still running: stop the I/O thread before it is destroyed
        if (io.joinable()) {
            stopping.store(true);
            uint64_t one = 1;
            if (wake >= 0) {
                ssize_t r = write(wake, &one, sizeof one);
                (void)r;
            }
            io.join();
        }
    }
    // counters (read through bfront_stats)
    uint64_t n_accepted = 0, n_requests = 0, n_stream_events = 0, n_stream_tokens = 0, n_idle_closed = 0;
    std::atomic<uint64_t> n_bytes_out{0};
};

// ---- small helpers ------------------------------------------------------------------------------------------------------
static void set_nonblock(int fd) { fcntl(fd, F_SETFL, fcntl(fd, F_GETFL, 0) | O_NONBLOCK); }

static const char* reason(int status) {
    switch (status) {
        case 100: return "Continue";
        case 200: return "OK";
        case 201: return "Created";
        case 204: return "No Content";
        case 400: return "Bad Request";
        case 401: return "Unauthorized";
        case 403: return "Forbidden";
        case 404: return "Not Found";
        case 405: return "Method Not Allowed";
        case 408: return "Request Timeout";
        case 413: return "Payload Too Large";
        case 422: return "Unprocessable Entity";
        case 429: return "Too Many Requests";
        case 431: return "Request Header Fields Too Large";
        case 500: return "Internal Server Error";
        case 501: return "Not Implemented";
        case 503: return "Service Unavailable";
        case 504: return "Gateway Timeout";
        default: return "Status";
    }
}

static bool ieq(const char* a, size_t n, const char* lit) {
    size_t m = strlen(lit);
    if (n != m) return false;
    for (size_t i = 0; i < n; ++i) {
        char c = a[i];
        if (c >= 'A' && c <= 'Z') c = char(c - 'A' + 'a');
        if (c != lit[i]) return false;
    }
    return true;
}

static void json_escape(const char* s, size_t n, std::string& out) {
    static const char* hex = "0123456789abcdef";
    for (size_t i = 0; i < n; ++i) {
        unsigned char c = (unsigned char)s[i];
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if (c < 0x20) {
                    out += "\\u00";
                    out += hex[c >> 4];
                    out += hex[c & 15];
                } else {
                    out += char(c);
                }
        }
    }
}

// Appends s[0, n) with ill-formed UTF-8 replaced by U+FFFD, one per maximal ill-formed subsequence (a truncated
// character is one replacement, as in Python's ``errors="replace"``).
static void utf8_sanitize(const char* s, size_t n, std::string& out) {
    size_t i = 0;
    while (i < n) {
        unsigned char c = (unsigned char)s[i];
        if (c < 0x80) {
            out += char(c);
            ++i;
            continue;
        }
        size_t need = 0;
        unsigned char lo = 0x80, hi = 0xBF;                 // allowed range of the second byte
        if (c >= 0xC2 && c <= 0xDF) {
            need = 2;
        } else if (c >= 0xE0 && c <= 0xEF) {
            need = 3;
            if (c == 0xE0) lo = 0xA0;                       // no overlong forms
            if (c == 0xED) hi = 0x9F;                       // no surrogates
        } else if (c >= 0xF0 && c <= 0xF4) {
            need = 4;
            if (c == 0xF0) lo = 0x90;
            if (c == 0xF4) hi = 0x8F;                       // nothing above U+10FFFF
        }
        if (need == 0) {
            out += "\xEF\xBF\xBD";
            ++i;
            continue;
        }
        size_t k = 1;
        while (k < need && i + k < n) {
            unsigned char d = (unsigned char)s[i + k];
            if (d < (k == 1 ? lo : 0x80) || d > (k == 1 ? hi : 0xBF)) break;
            ++k;
        }
        if (k == need) {
            out.append(s + i, need);
        } else {
            out += "\xEF\xBF\xBD";
        }
        i += k;
    }
}

// Length of the longest prefix of s[0, n) that does not end inside a UTF-8 sequence.
static size_t utf8_complete_prefix(const char* s, size_t n) {
    for (size_t back = 1; back <= 4 && back <= n; ++back) {
        unsigned char c = (unsigned char)s[n - back];
        if ((c & 0xC0) == 0x80) continue;
        size_t need = c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 1;
        return need > back ? n - back : n;
    }
    return n;
}

static void wake_io(Front* f) {
    if (f->stopping.load(std::memory_order_relaxed)) return;
    if (!f->wake_pending.exchange(true)) {
        uint64_t one = 1;
        ssize_t r = write(f->wake, &one, sizeof one);
        (void)r;
    }
}

// Output goes to the connection's buffer; the I/O thread sends it.  Caller holds f->mu.
static bool queue_out(Front* f, Conn* c, const char* data, size_t n) {
    if (c->out.size() + n > kMaxOut) {
        c->close_after_flush = true;
        return false;
    }
    c->out.append(data, n);
    f->dirty.push_back(c->id);
    return true;
}

static void append_chunk(std::string& out, const std::string& payload, bool raw = false) {
    if (raw) {
        out += payload;
        return;
    }
    char len[24];
    int k = snprintf(len, sizeof len, "%zx\r\n", payload.size());
    out.append(len, size_t(k));
    out += payload;
    out += "\r\n";
}

// ---- token streams ---------------------------------------------------------------------------------------------------------
static void stream_event_text(Stream* s, const char* text, size_t n, std::string& framed) {
    std::string ev;
    ev.reserve(s->head.size() + n + 64);
    ev += "data: ";
    ev += s->head;
    ev += s->chat ? "\"delta\": {\"content\": \"" : "\"text\": \"";
    std::string clean;
    utf8_sanitize(text, n, clean);
    json_escape(clean.data(), clean.size(), ev);
    ev += s->chat ? "\"}, \"finish_reason\": null}]}\n\n" : "\", \"finish_reason\": null}]}\n\n";
    append_chunk(framed, ev, s->raw);
    s->events++;
}

// Sends (or parks, before the head is out) framed bytes of a stream.  Caller holds f->mu.
static void stream_emit(Front* f, Stream* s, const std::string& framed) {
    if (framed.empty()) return;
    if (!s->begun) {
        s->early += framed;
        return;
    }
    auto it = f->conns.find(s->conn);
    if (it == f->conns.end()) {
        if (s->state == LIVE) s->state = CLIENT_GONE;
        return;
    }
    if (!queue_out(f, it->second.get(), framed.data(), framed.size()) && s->state == LIVE) s->state = CLIENT_GONE;
}

// Appends the decoded bytes of a token and frames what has become safe to send.  Returns the stream's state.
static int stream_feed(Front* f, Stream* s, const uint8_t* bytes, size_t n, std::string& framed) {
    s->held.append(reinterpret_cast<const char*>(bytes), n);
    const std::string& h = s->held;
    size_t valid = utf8_complete_prefix(h.data(), h.size());
    // a stop sequence inside the text that has not gone out yet ends the stream in front of it
    size_t hit = std::string::npos;
    for (const std::string& st : s->stops) {
        if (st.empty()) continue;
        size_t p = h.find(st);
        if (p != std::string::npos && p + st.size() <= valid && p < hit) hit = p;
    }
    if (hit != std::string::npos) {
        if (hit > 0) stream_event_text(s, h.data(), hit, framed);
        s->held.clear();
        s->state = STOP_HIT;
        return s->state;
    }
    // text that may still turn into a stop sequence is held back
    size_t hold = 0;
    for (const std::string& st : s->stops) {
        size_t maxl = st.size() > 0 ? st.size() - 1 : 0;
        if (maxl > valid) maxl = valid;
        for (size_t L = maxl; L > 0; --L) {
            if (memcmp(h.data() + valid - L, st.data(), L) == 0) {
                if (L > hold) hold = L;
                break;
            }
        }
    }
    size_t safe = valid - hold;
    // never cut inside a character: the held part starts at a character boundary
    while (safe > 0 && safe < h.size() && (((unsigned char)h[safe]) & 0xC0) == 0x80) --safe;
    if (safe > 0) {
        stream_event_text(s, h.data(), safe, framed);
        s->held.erase(0, safe);
    }
    (void)f;
    return s->state;
}

// ---- connections (I/O thread) -------------------------------------------------------------------------------------------------
static void epoll_set(Front* f, Conn* c, bool want_write) {
    epoll_event ev{};
    ev.events = uint32_t(EPOLLIN) | uint32_t(EPOLLRDHUP) | (want_write ? uint32_t(EPOLLOUT) : 0u);
    ev.data.u64 = uint64_t(c->id);
    epoll_ctl(f->ep, EPOLL_CTL_MOD, c->fd, &ev);
    c->want_write = want_write;
}

// Caller holds f->mu.  The connection object is gone afterwards.
static void close_conn(Front* f, int64_t id) {
    auto it = f->conns.find(id);
    if (it == f->conns.end()) return;
    Conn* c = it->second.get();
    if (c->stream) {
        auto st = f->streams.find(c->stream);
        if (st != f->streams.end() && st->second->state == LIVE) st->second->state = CLIENT_GONE;
    }
    if (c->state != READING) {                 // somebody is working on this connection's request: tell them
        Event e;
        e.kind = 2;
        e.conn = id;
        f->events.push_back(std::move(e));
        f->cv.notify_one();
    }
    epoll_ctl(f->ep, EPOLL_CTL_DEL, c->fd, nullptr);
    close(c->fd);
    f->conns.erase(it);
}

static void simple_response(Front* f, Conn* c, int status, const char* text) {
    char buf[512];
    int n = snprintf(buf, sizeof buf, "HTTP/1.1 %d %s\r\ncontent-type: text/plain\r\ncontent-length: %zu\r\nconnection: close\r\n\r\n%s",
                     status, reason(status), strlen(text), text);
    c->out.append(buf, size_t(n));
    c->close_after_flush = true;
    (void)f;
}

// Tries to cut one request off the front of c->in.  Caller holds f->mu.  Returns false when the connection was closed.
static bool try_parse(Front* f, Conn* c) {
    while (c->state == READING && !c->close_after_flush) {
        size_t he = c->in.find("\r\n\r\n");
        if (he == std::string::npos) {
            if (c->in.size() > kMaxHeader) simple_response(f, c, 431, "header too large");
            return true;
        }
        if (he > kMaxHeader) {
            simple_response(f, c, 431, "header too large");
            return true;
        }
        const char* p = c->in.data();
        size_t le = c->in.find("\r\n");
        // request line
        size_t sp1 = c->in.find(' ');
        size_t sp2 = sp1 == std::string::npos ? std::string::npos : c->in.find(' ', sp1 + 1);
        if (sp1 == std::string::npos || sp2 == std::string::npos || sp2 > le) {
            simple_response(f, c, 400, "malformed request line");
            return true;
        }
        std::string method(p, sp1), target(p + sp1 + 1, sp2 - sp1 - 1), version(p + sp2 + 1, le - sp2 - 1);
        bool http10 = version == "HTTP/1.0";
        if (version != "HTTP/1.1" && !http10) {
            simple_response(f, c, 400, "unsupported HTTP version");
            return true;
        }
        size_t content_length = 0;
        bool chunked = false, expect = false, keep = !http10, have_length = false;
        size_t pos = le + 2;
        while (pos < he + 2) {
            size_t eol = c->in.find("\r\n", pos);
            size_t colon = c->in.find(':', pos);
            if (colon == std::string::npos || colon > eol) {
                simple_response(f, c, 400, "malformed header");
                return true;
            }
            size_t vs = colon + 1;
            while (vs < eol && (p[vs] == ' ' || p[vs] == '\t')) ++vs;
            size_t ve = eol;
            while (ve > vs && (p[ve - 1] == ' ' || p[ve - 1] == '\t')) --ve;
            const char* name = p + pos;
            size_t nlen = colon - pos;
            if (ieq(name, nlen, "content-length")) {
                const size_t previous = content_length;
                const bool repeated = have_length;
                have_length = true;
                content_length = 0;
                if (ve == vs) {
                    simple_response(f, c, 400, "bad content-length");
                    return true;
                }
                for (size_t i = vs; i < ve; ++i) {
                    if (p[i] < '0' || p[i] > '9' || content_length > kMaxBody) {
                        simple_response(f, c, 400, "bad content-length");
                        return true;
                    }
                    content_length = content_length * 10 + size_t(p[i] - '0');
                }
                if (repeated && previous != content_length) {                     // two lengths that disagree: refuse, do not guess
                    simple_response(f, c, 400, "conflicting content-length headers");
                    return true;
                }
            } else if (ieq(name, nlen, "transfer-encoding")) {
                chunked = !ieq(p + vs, ve - vs, "identity");
            } else if (ieq(name, nlen, "expect")) {
                expect = ieq(p + vs, ve - vs, "100-continue");
            } else if (ieq(name, nlen, "connection")) {
                if (ieq(p + vs, ve - vs, "close")) keep = false;
                if (ieq(p + vs, ve - vs, "keep-alive")) keep = true;
            }
            pos = eol + 2;
        }
        if (content_length > kMaxBody) {
            simple_response(f, c, 413, "body too large");
            return true;
        }
        auto want_more = [&]() {                         // the request is not complete yet
            if (expect && !c->continued) {
                c->out += "HTTP/1.1 100 Continue\r\n\r\n";
                c->continued = true;
            }
        };
        std::string body;
        size_t total;
        if (chunked) {
            // chunked transfer coding: "<hex size>[;extensions]\r\n<data>\r\n" ... "0\r\n" [trailers] "\r\n"
            size_t q = he + 4;
            bool done = false, bad = false;
            while (!done) {
                size_t eol = c->in.find("\r\n", q);
                if (eol == std::string::npos) break;
                size_t size = 0, digits = 0;
                for (size_t i = q; i < eol && p[i] != ';'; ++i) {
                    const char ch = p[i];
                    int v = ch >= '0' && ch <= '9' ? ch - '0' : ch >= 'a' && ch <= 'f' ? ch - 'a' + 10 : ch >= 'A' && ch <= 'F' ? ch - 'A' + 10 : -1;
                    if (v < 0 || ++digits > 8) {
                        bad = true;
                        break;
                    }
                    size = size * 16 + size_t(v);
                }
                if (bad || digits == 0 || body.size() + size > kMaxBody) {
                    bad = true;
                    break;
                }
                if (size == 0) {                                     // last chunk: skip the trailer section up to the blank line
                    size_t t = eol + 2;
                    while (true) {
                        size_t e2 = c->in.find("\r\n", t);
                        if (e2 == std::string::npos) break;
                        if (e2 == t) {
                            q = e2 + 2;
                            done = true;
                            break;
                        }
                        t = e2 + 2;
                    }
                    break;
                }
                if (c->in.size() < eol + 2 + size + 2) break;
                if (p[eol + 2 + size] != '\r' || p[eol + 2 + size + 1] != '\n') {
                    bad = true;
                    break;
                }
                body.append(p + eol + 2, size);
                q = eol + 2 + size + 2;
            }
            if (bad) {
                simple_response(f, c, body.size() > kMaxBody / 2 ? 413 : 400, "malformed chunked body");
                return true;
            }
            if (!done) {
                want_more();
                return true;
            }
            total = q;
        } else {
            total = he + 4 + content_length;
            if (c->in.size() < total) {
                want_more();
                return true;
            }
            body.assign(p + he + 4, content_length);
        }
        Event e;
        e.kind = 1;
        e.conn = c->id;
        e.method = std::move(method);
        e.target = std::move(target);
        e.headers.assign(p + le + 2, he + 2 - (le + 2));
        e.body = std::move(body);
        e.peer = c->peer;
        c->in.erase(0, total);
        c->keep_alive = keep;
        c->continued = false;
        c->head_only = e.method == "HEAD";
        c->http10 = http10;
        c->state = DISPATCHED;
        f->n_requests++;
        f->events.push_back(std::move(e));
        f->cv.notify_one();
    }
    return true;
}

// Sends what is buffered.  I/O thread, mutex not held.  Returns false when the connection was closed.
static bool flush_conn(Front* f, Conn* c) {
    while (true) {
        if (c->wire_off == c->wire.size()) {
            c->wire.clear();
            c->wire_off = 0;
            bool closing;
            {
                std::lock_guard<std::mutex> lk(f->mu);
                c->wire.swap(c->out);
                closing = c->close_after_flush;
                if (c->wire.empty() && closing) {
                    close_conn(f, c->id);
                    return false;
                }
            }
            if (c->wire.empty()) {
                if (c->want_write) epoll_set(f, c, false);
                return true;
            }
        }
        ssize_t n = send(c->fd, c->wire.data() + c->wire_off, c->wire.size() - c->wire_off, MSG_NOSIGNAL);
        if (n > 0) {
            c->last_io = Clock::now();
            c->wire_off += size_t(n);
            f->n_bytes_out.fetch_add(uint64_t(n), std::memory_order_relaxed);
            continue;
        }
        if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) {
            if (!c->want_write) epoll_set(f, c, true);
            return true;
        }
        if (n < 0 && errno == EINTR) continue;
        std::lock_guard<std::mutex> lk(f->mu);
        close_conn(f, c->id);
        return false;
    }
}

// A response has been written completely: back to reading (or close).  Caller holds f->mu (any thread).
static void response_done(Front* f, Conn* c) {
    c->stream = 0;
    if (!c->keep_alive) {
        c->close_after_flush = true;
    } else {
        c->state = READING;
        c->reparse = true;                      // the I/O thread looks for a pipelined request
    }
    f->dirty.push_back(c->id);
}

static Conn* find_conn(Front* f, int64_t id) {
    std::lock_guard<std::mutex> lk(f->mu);
    auto it = f->conns.find(id);
    return it == f->conns.end() ? nullptr : it->second.get();      // stable: only the I/O thread erases connections
}

// "address:port" of a client; an IPv4 client of a dual-stack socket is named by its IPv4 address.
std::string peer_name(const sockaddr_storage& ss) {
    char ip[INET6_ADDRSTRLEN] = "";
    int port = 0;
    if (ss.ss_family == AF_INET6) {
        const auto* a = reinterpret_cast<const sockaddr_in6*>(&ss);
        port = ntohs(a->sin6_port);
        if (IN6_IS_ADDR_V4MAPPED(&a->sin6_addr))
            inet_ntop(AF_INET, a->sin6_addr.s6_addr + 12, ip, sizeof ip);
        else
            inet_ntop(AF_INET6, &a->sin6_addr, ip, sizeof ip);
    } else {
        const auto* a = reinterpret_cast<const sockaddr_in*>(&ss);
        port = ntohs(a->sin_port);
        inet_ntop(AF_INET, &a->sin_addr, ip, sizeof ip);
    }
    return std::string(ip) + ":" + std::to_string(port);
}

static void io_loop(Front* f) {
    std::vector<epoll_event> evs(256);
    std::vector<char> buf(1 << 16);
    auto last_sweep = Clock::now();
    while (!f->stopping.load()) {
        int n = epoll_wait(f->ep, evs.data(), int(evs.size()), f->lazy.load(std::memory_order_relaxed) ? 5 : 200);
        if (n < 0 && errno != EINTR) break;
        for (int i = 0; i < n; ++i) {
            uint64_t tag = evs[i].data.u64;
            if (tag == 0) {                                                       // the listening socket
                while (true) {
                    sockaddr_storage addr{};
                    socklen_t al = sizeof addr;
                    int fd = accept4(f->listen_fd, reinterpret_cast<sockaddr*>(&addr), &al, SOCK_NONBLOCK | SOCK_CLOEXEC);
                    if (fd < 0) break;
                    int one = 1;
                    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
                    auto c = std::make_unique<Conn>();
                    c->fd = fd;
                    c->peer = peer_name(addr);
                    std::lock_guard<std::mutex> lk(f->mu);
                    c->id = f->next_id++;
                    epoll_event ev{};
                    ev.events = EPOLLIN | EPOLLRDHUP;
                    ev.data.u64 = uint64_t(c->id);
                    epoll_ctl(f->ep, EPOLL_CTL_ADD, fd, &ev);
                    f->n_accepted++;
                    f->conns.emplace(c->id, std::move(c));
                }
                continue;
            }
            if (tag == UINT64_MAX) {                                              // woken by another thread
                uint64_t v;
                ssize_t r = read(f->wake, &v, sizeof v);
                (void)r;
                f->wake_pending.store(false);
                continue;
            }
            Conn* c = find_conn(f, int64_t(tag));
            if (!c) continue;
            uint32_t e = evs[i].events;
            bool alive = true;
            if (e & EPOLLIN) {
                while (alive) {
                    ssize_t r = recv(c->fd, buf.data(), buf.size(), 0);
                    if (r > 0) {
                        c->last_io = Clock::now();
                        if (c->in.size() + size_t(r) > kMaxBody + kMaxHeader) {
                            alive = false;
                            break;
                        }
                        c->in.append(buf.data(), size_t(r));
                        continue;
                    }
                    if (r < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) break;
                    if (r < 0 && errno == EINTR) continue;
                    alive = false;                                                // orderly shutdown by the peer, or an error
                }
                if (alive) {
                    {
                        std::lock_guard<std::mutex> lk(f->mu);
                        try_parse(f, c);
                    }
                    alive = flush_conn(f, c);
                    if (!alive) continue;
                }
            }
            if (alive && (e & (EPOLLHUP | EPOLLERR))) alive = false;
            if (alive && (e & EPOLLRDHUP) && !(e & EPOLLIN)) alive = false;
            if (!alive) {
                std::lock_guard<std::mutex> lk(f->mu);
                close_conn(f, c->id);
                continue;
            }
            if (e & EPOLLOUT) flush_conn(f, c);
        }
        // output queued (or responses completed) by other threads
        std::vector<int64_t> d;
        {
            std::lock_guard<std::mutex> lk(f->mu);
            d.swap(f->dirty);
        }
        for (int64_t id : d) {
            Conn* c = find_conn(f, id);
            if (!c) continue;
            bool again;
            {
                std::lock_guard<std::mutex> lk(f->mu);
                again = c->reparse;
                c->reparse = false;
                if (again) try_parse(f, c);
            }
            flush_conn(f, c);
        }
        // streams past their deadline
        auto now = Clock::now();
        if (now - last_sweep > std::chrono::milliseconds(100)) {
            last_sweep = now;
            std::lock_guard<std::mutex> lk(f->mu);
            for (auto& kv : f->streams) {
                Stream* s = kv.second.get();
                if (s->state == LIVE && s->has_deadline && now > s->deadline) s->state = TIMED_OUT;
            }
            // connections that wait for a request (or sit on half of one) without moving a byte
            const int idle_ms = f->idle_timeout_ms.load(std::memory_order_relaxed);
            if (idle_ms > 0) {
                std::vector<int64_t> idle;
                for (auto& kv : f->conns) {
                    Conn* c = kv.second.get();
                    if (c->state == READING && now - c->last_io > std::chrono::milliseconds(idle_ms)) idle.push_back(c->id);
                }
                for (int64_t id : idle) close_conn(f, id);
                f->n_idle_closed += idle.size();
            }
        }
    }
}

}  // namespace bonsai_front

// ---- C ABI ----------------------------------------------------------------------------------------------------------------
using namespace bonsai_front;

extern "C" {

// Binds and listens (port 0: the kernel picks one).  Returns nullptr when the address cannot be bound.
void* bfront_create(const char* host, int port, int backlog) {
    auto f = std::make_unique<Front>();
    f->host = host ? host : "127.0.0.1";
    // A literal address of either family or a name; a name's IPv4 addresses are tried first (clients of "localhost" mostly
    // dial 127.0.0.1), and "::" listens on both families.
    addrinfo hints{};
    hints.ai_family = AF_UNSPEC;
    hints.ai_socktype = SOCK_STREAM;
    hints.ai_flags = AI_PASSIVE | AI_NUMERICSERV;
    addrinfo* res = nullptr;
    const std::string service = std::to_string(port);
    if (getaddrinfo(f->host.empty() ? nullptr : f->host.c_str(), service.c_str(), &hints, &res) != 0 || res == nullptr) return nullptr;
    f->listen_fd = -1;
    for (int family : {AF_INET, AF_INET6}) {
        for (addrinfo* ai = res; ai != nullptr && f->listen_fd < 0; ai = ai->ai_next) {
            if (ai->ai_family != family) continue;
            int fd = socket(ai->ai_family, SOCK_STREAM | SOCK_CLOEXEC, 0);
            if (fd < 0) continue;
            int one = 1, zero = 0;
            setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
            if (family == AF_INET6) setsockopt(fd, IPPROTO_IPV6, IPV6_V6ONLY, f->host == "::" ? &zero : &one, sizeof one);
            if (bind(fd, ai->ai_addr, ai->ai_addrlen) == 0 && listen(fd, backlog > 0 ? backlog : 1024) == 0)
                f->listen_fd = fd;
            else
                close(fd);
        }
    }
    freeaddrinfo(res);
    if (f->listen_fd < 0) return nullptr;
    sockaddr_storage bound{};
    socklen_t al = sizeof bound;
    getsockname(f->listen_fd, reinterpret_cast<sockaddr*>(&bound), &al);
    f->port = ntohs(bound.ss_family == AF_INET6 ? reinterpret_cast<sockaddr_in6*>(&bound)->sin6_port : reinterpret_cast<sockaddr_in*>(&bound)->sin_port);
    set_nonblock(f->listen_fd);
    f->ep = epoll_create1(EPOLL_CLOEXEC);
    f->wake = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
    epoll_event ev{};
    ev.events = EPOLLIN;
    ev.data.u64 = 0;
    epoll_ctl(f->ep, EPOLL_CTL_ADD, f->listen_fd, &ev);
    ev.data.u64 = UINT64_MAX;
    epoll_ctl(f->ep, EPOLL_CTL_ADD, f->wake, &ev);
    static std::mutex reg_mu;
    static std::vector<std::unique_ptr<Front>> registry;      // fronts live as long as the process (see bfront_destroy)
    std::lock_guard<std::mutex> lk(reg_mu);
    registry.push_back(std::move(f));
    return registry.back().get();
}

int bfront_port(void* h) { return static_cast<Front*>(h)->port; }

int bfront_start(void* h) {
    Front* f = static_cast<Front*>(h);
    if (f->io.joinable()) return 0;
    f->io = std::thread(io_loop, f);
    return 0;
}

void bfront_stop(void* h) {
    Front* f = static_cast<Front*>(h);
    if (f->stopping.exchange(true)) return;
    uint64_t one = 1;
    ssize_t r = write(f->wake, &one, sizeof one);       // wake_io() is a no-op once the front is stopping
    (void)r;
    if (f->io.joinable()) f->io.join();
    std::lock_guard<std::mutex> lk(f->mu);
    for (auto& kv : f->conns) close(kv.second->fd);
    f->conns.clear();
    for (auto& kv : f->streams)
        if (kv.second->state == LIVE) kv.second->state = CLIENT_GONE;
    if (f->listen_fd >= 0) close(f->listen_fd);
    f->listen_fd = -1;
    f->cv.notify_all();
}

// Stops the front and releases its descriptors.  The object itself stays valid until the process ends: a scheduler thread
// may still push a token, and an event waiter may still be on its way out, after the owner has closed the front; every
// call on a stopped front returns "gone" instead of touching freed memory.
void bfront_destroy(void* h) {
    Front* f = static_cast<Front*>(h);
    bfront_stop(h);
    std::lock_guard<std::mutex> lk(f->mu);
    if (f->ep >= 0) close(f->ep);
    if (f->wake >= 0) close(f->wake);
    f->ep = f->wake = -1;
    f->streams.clear();
    f->events.clear();
    f->vocab_bytes.clear();
    f->vocab_bytes.shrink_to_fit();
}

// Token id -> bytes table: ``offsets`` has n + 1 entries into ``bytes``.
void bfront_set_vocab(void* h, const uint8_t* bytes, const uint32_t* offsets, uint32_t n) {
    Front* f = static_cast<Front*>(h);
    std::lock_guard<std::mutex> lk(f->mu);
    f->vocab_off.assign(offsets, offsets + n + 1);
    f->vocab_bytes.assign(bytes, bytes + offsets[n]);
}

// Blocks up to timeout_ms for a request or a disconnect notice.  Returns a malloc'd record (free it with bfront_free):
//   int32 kind (1 request, 2 connection closed) | int64 conn | uint32 lengths[5] (method, target, headers, body, peer) | the bytes
// or nullptr on time-out; *stopped is set when the front has been stopped.
void* bfront_next_event(void* h, int timeout_ms, int* stopped) {
    Front* f = static_cast<Front*>(h);
    std::unique_lock<std::mutex> lk(f->mu);
    if (f->events.empty())
        f->cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return !f->events.empty() || f->stopping.load(); });
    if (stopped) *stopped = f->stopping.load() ? 1 : 0;
    if (f->events.empty()) return nullptr;
    Event e = std::move(f->events.front());
    f->events.pop_front();
    lk.unlock();
    const std::string* parts[5] = {&e.method, &e.target, &e.headers, &e.body, &e.peer};
    size_t total = 4 + 8 + 5 * 4;
    for (auto* p : parts) total += p->size();
    char* rec = static_cast<char*>(malloc(total));
    if (!rec) return nullptr;
    int32_t kind = e.kind;
    memcpy(rec, &kind, 4);
    memcpy(rec + 4, &e.conn, 8);
    size_t off = 12 + 20;
    for (int i = 0; i < 5; ++i) {
        uint32_t n = uint32_t(parts[i]->size());
        memcpy(rec + 12 + 4 * i, &n, 4);
        memcpy(rec + off, parts[i]->data(), n);
        off += n;
    }
    return rec;
}

void bfront_free(void* p) { free(p); }

// A complete response (content-length framing).  ``headers`` is a block of "name: value\r\n" lines.
int bfront_respond(void* h, int64_t conn, int status, const char* headers, const uint8_t* body, uint64_t n) {
    Front* f = static_cast<Front*>(h);
    std::lock_guard<std::mutex> lk(f->mu);
    auto it = f->conns.find(conn);
    if (it == f->conns.end() || it->second->state != DISPATCHED) return -1;
    Conn* c = it->second.get();
    char line[128];
    int k = snprintf(line, sizeof line, "HTTP/1.1 %d %s\r\n", status, reason(status));
    std::string head(line, size_t(k));
    head += headers ? headers : "";
    k = snprintf(line, sizeof line, "content-length: %llu\r\n%s\r\n", static_cast<unsigned long long>(n), c->keep_alive ? "" : "connection: close\r\n");
    head.append(line, size_t(k));
    queue_out(f, c, head.data(), head.size());
    if (n && !c->head_only) queue_out(f, c, reinterpret_cast<const char*>(body), size_t(n));
    response_done(f, c);
    wake_io(f);
    return 0;
}

// A response whose body follows in pieces (chunked transfer encoding).
int bfront_respond_start(void* h, int64_t conn, int status, const char* headers) {
    Front* f = static_cast<Front*>(h);
    std::lock_guard<std::mutex> lk(f->mu);
    auto it = f->conns.find(conn);
    if (it == f->conns.end() || it->second->state != DISPATCHED) return -1;
    Conn* c = it->second.get();
    char line[128];
    int k = snprintf(line, sizeof line, "HTTP/1.1 %d %s\r\n", status, reason(status));
    std::string head(line, size_t(k));
    head += headers ? headers : "";
    if (c->http10) c->keep_alive = false;                   // the end of the body is the end of the connection
    else head += "transfer-encoding: chunked\r\n";
    if (!c->keep_alive) head += "connection: close\r\n";
    head += "\r\n";
    c->state = RESPONDING;
    queue_out(f, c, head.data(), head.size());
    wake_io(f);
    return 0;
}

int bfront_respond_chunk(void* h, int64_t conn, const uint8_t* data, uint64_t n) {
    Front* f = static_cast<Front*>(h);
    if (n == 0) return 0;
    std::lock_guard<std::mutex> lk(f->mu);
    auto it = f->conns.find(conn);
    if (it == f->conns.end() || it->second->state != RESPONDING) return -1;
    if (it->second->head_only) return 0;
    std::string framed;
    append_chunk(framed, std::string(reinterpret_cast<const char*>(data), size_t(n)), it->second->http10);
    bool ok = queue_out(f, it->second.get(), framed.data(), framed.size());
    wake_io(f);
    return ok ? 0 : -1;
}

int bfront_respond_end(void* h, int64_t conn) {
    Front* f = static_cast<Front*>(h);
    std::lock_guard<std::mutex> lk(f->mu);
    auto it = f->conns.find(conn);
    if (it == f->conns.end() || it->second->state != RESPONDING) return -1;
    Conn* c = it->second.get();
    if (!c->head_only && !c->http10) queue_out(f, c, "0\r\n\r\n", 5);
    response_done(f, c);
    wake_io(f);
    return 0;
}

// Opens a token stream on a dispatched connection.  ``chunk_head``: the JSON text every chunk starts with, up to and
// including ``"choices": [{"index": 0, `` ; ``stops``: uint32 count, then per stop sequence uint32 length + bytes;
// ``first_event``: complete SSE event sent before the first token (the role chunk), may be empty.  Tokens may be pushed
// at once; their events are parked until bfront_stream_begin() has written the response head.
int64_t bfront_stream_open(void* h, int64_t conn, const char* chunk_head, int chat, const uint8_t* stops, const char* first_event, int timeout_ms) {
    Front* f = static_cast<Front*>(h);
    std::lock_guard<std::mutex> lk(f->mu);
    auto it = f->conns.find(conn);
    if (it == f->conns.end() || it->second->state != DISPATCHED || it->second->stream) return -1;
    auto s = std::make_unique<Stream>();
    s->id = f->next_id++;
    s->conn = conn;
    s->head = chunk_head;
    s->chat = chat != 0;
    if (stops) {
        uint32_t count;
        memcpy(&count, stops, 4);
        size_t off = 4;
        for (uint32_t i = 0; i < count; ++i) {
            uint32_t len;
            memcpy(&len, stops + off, 4);
            off += 4;
            s->stops.emplace_back(reinterpret_cast<const char*>(stops + off), len);
            off += len;
        }
    }
    s->raw = it->second->http10;
    if (first_event && *first_event) append_chunk(s->early, first_event, s->raw);
    if (timeout_ms > 0) {
        s->deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
        s->has_deadline = true;
    }
    int64_t id = s->id;
    it->second->stream = id;
    f->streams.emplace(id, std::move(s));
    return id;
}

// Writes the response head of a stream (status 200, chunked, plus ``headers``) and releases the parked events.
int bfront_stream_begin(void* h, int64_t stream, const char* headers) {
    Front* f = static_cast<Front*>(h);
    std::lock_guard<std::mutex> lk(f->mu);
    auto st = f->streams.find(stream);
    if (st == f->streams.end()) return -1;
    Stream* s = st->second.get();
    auto it = f->conns.find(s->conn);
    if (it == f->conns.end() || it->second->state != DISPATCHED) {       // the client left before the head was written
        s->begun = true;
        s->early.clear();
        if (s->state == FINISHED) {
            f->streams.erase(st);
        } else if (s->state == LIVE) {
            s->state = CLIENT_GONE;
        }
        return -1;
    }
    Conn* c = it->second.get();
    std::string head = "HTTP/1.1 200 OK\r\n";
    head += headers ? headers : "";
    if (c->http10) c->keep_alive = false;
    else head += "transfer-encoding: chunked\r\n";
    if (!c->keep_alive) head += "connection: close\r\n";
    head += "\r\n";
    c->state = STREAMING;
    s->begun = true;
    queue_out(f, c, head.data(), head.size());
    if (!s->early.empty()) {
        queue_out(f, c, s->early.data(), s->early.size());
        s->early.clear();
        s->early.shrink_to_fit();
    }
    if (s->state == FINISHED) {                      // the generation ended before the head was written
        response_done(f, c);
        f->streams.erase(st);
    }
    wake_io(f);
    return 0;
}

// One sampled token.  Returns the stream's state: 0 live, 1 a stop sequence was hit (nothing after it is sent), 2 the
// client is gone, 3 the request's time is up, -1 unknown stream.  Any non-zero value asks the caller to stop generating.
int bfront_stream_push(void* h, int64_t stream, int32_t token) {
    Front* f = static_cast<Front*>(h);
    std::lock_guard<std::mutex> lk(f->mu);
    auto st = f->streams.find(stream);
    if (st == f->streams.end()) return -1;
    Stream* s = st->second.get();
    if (s->state != LIVE) return s->state;
    if (token < 0 || size_t(token) + 1 >= f->vocab_off.size()) return 0;          // an id without bytes adds no text
    uint32_t a = f->vocab_off[size_t(token)], b = f->vocab_off[size_t(token) + 1];
    s->tokens++;
    f->n_stream_tokens++;
    std::string framed;
    uint64_t before = s->events;
    stream_feed(f, s, f->vocab_bytes.data() + a, b - a, framed);
    f->n_stream_events += s->events - before;
    if (!framed.empty()) {
        stream_emit(f, s, framed);
        if (s->begun && !f->lazy.load(std::memory_order_relaxed)) wake_io(f);
    }
    return s->state;
}

// With lazy wake-ups on, bfront_stream_push() only queues; the producer calls bfront_kick() after the tokens of a decode
// step (one wake-up and one pass over the connections per step instead of one per token).  The I/O thread still looks at
// the queue every few milliseconds, so a missing kick delays output, it does not lose it.
void bfront_set_lazy(void* h, int on) { static_cast<Front*>(h)->lazy.store(on != 0); }

void bfront_kick(void* h) { wake_io(static_cast<Front*>(h)); }

// Connections that wait for a request without receiving or sending a byte for this long are closed (0: never).  Connections
// whose request is being answered or streamed are not subject to it.
void bfront_set_idle_timeout(void* h, int milliseconds) { static_cast<Front*>(h)->idle_timeout_ms.store(milliseconds < 0 ? 0 : milliseconds); }

// Ends a stream: the held-back text (unless a stop sequence was hit), the finish chunk, "[DONE]" and the terminating chunk;
// with ``error`` an error event instead.  The connection goes back to reading requests.  Returns the number of tokens pushed.
int64_t bfront_stream_finish(void* h, int64_t stream, const char* finish_reason, const char* error) {
    Front* f = static_cast<Front*>(h);
    std::lock_guard<std::mutex> lk(f->mu);
    auto st = f->streams.find(stream);
    if (st == f->streams.end()) return -1;
    Stream* s = st->second.get();
    int64_t ntok = int64_t(s->tokens);
    std::string framed;
    if (error && *error) {
        std::string ev = "data: {\"error\": {\"message\": \"";
        std::string clean;
        utf8_sanitize(error, strlen(error), clean);
        json_escape(clean.data(), clean.size(), ev);
        ev += "\", \"type\": \"server_error\"}}\n\n";
        append_chunk(framed, ev, s->raw);
    } else {
        bool stop_hit = s->state == STOP_HIT;
        if (!stop_hit && !s->held.empty()) stream_event_text(s, s->held.data(), s->held.size(), framed);
        s->held.clear();
        std::string ev = "data: ";
        ev += s->head;
        ev += s->chat ? "\"delta\": {}, \"finish_reason\": \"" : "\"text\": \"\", \"finish_reason\": \"";
        const char* fr = stop_hit ? "stop" : (finish_reason && *finish_reason ? finish_reason : "stop");
        json_escape(fr, strlen(fr), ev);
        ev += "\"}]}\n\n";
        append_chunk(framed, ev, s->raw);
        append_chunk(framed, "data: [DONE]\n\n", s->raw);
    }
    if (!s->raw) framed += "0\r\n\r\n";
    bool was_live_conn = s->state != CLIENT_GONE;
    stream_emit(f, s, framed);
    s->state = FINISHED;
    if (s->begun) {
        auto it = f->conns.find(s->conn);
        if (it != f->conns.end() && was_live_conn) response_done(f, it->second.get());
        f->streams.erase(st);
        wake_io(f);
    }                                                 // else: bfront_stream_begin() completes and erases it
    return ntok;
}

// Drops a stream that will never be begun (the request failed before a response head was chosen).
void bfront_stream_abandon(void* h, int64_t stream) {
    Front* f = static_cast<Front*>(h);
    std::lock_guard<std::mutex> lk(f->mu);
    auto st = f->streams.find(stream);
    if (st == f->streams.end()) return;
    auto it = f->conns.find(st->second->conn);
    if (it != f->conns.end()) it->second->stream = 0;
    f->streams.erase(st);
}

// out[0..7]: connections accepted, requests parsed, stream tokens, stream events, bytes written, open connections, open
// streams, connections closed for idleness.
void bfront_stats(void* h, uint64_t* out) {
    Front* f = static_cast<Front*>(h);
    std::lock_guard<std::mutex> lk(f->mu);
    out[0] = f->n_accepted;
    out[1] = f->n_requests;
    out[2] = f->n_stream_tokens;
    out[3] = f->n_stream_events;
    out[4] = f->n_bytes_out.load();
    out[5] = f->conns.size();
    out[6] = f->streams.size();
    out[7] = f->n_idle_closed;
}

}  // extern "C"
