// Race check of the HTTP / SSE front under ThreadSanitizer: compiled together with csrc/runtime/http_front.cpp by
// tests/test_native_front.py (g++ -fsanitize=thread).  Client threads open connections and read streams, a dispatcher
// thread answers requests and opens token streams, a producer thread pushes tokens into all open streams and kicks the I/O
// thread once per "step", one client leaves in mid-stream, and the front is closed while connections are still open.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

extern "C" {
void* bfront_create(const char*, int, int);
int bfront_port(void*);
int bfront_start(void*);
void bfront_stop(void*);
void bfront_destroy(void*);
void bfront_set_vocab(void*, const uint8_t*, const uint32_t*, uint32_t);
void* bfront_next_event(void*, int, int*);
void bfront_free(void*);
int bfront_respond(void*, int64_t, int, const char*, const uint8_t*, uint64_t);
int64_t bfront_stream_open(void*, int64_t, const char*, int, const uint8_t*, const char*, int);
int bfront_stream_begin(void*, int64_t, const char*);
int bfront_stream_push(void*, int64_t, int32_t);
int64_t bfront_stream_finish(void*, int64_t, const char*, const char*);
void bfront_set_lazy(void*, int);
void bfront_kick(void*);
void bfront_stats(void*, uint64_t*);
}

static int connect_to(int port) {
    int fd = socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons(uint16_t(port));
    inet_pton(AF_INET, "127.0.0.1", &a.sin_addr);
    if (connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof a) != 0) {
        close(fd);
        return -1;
    }
    return fd;
}

int main() {
    void* f = bfront_create("127.0.0.1", 0, 128);
    if (!f) return 2;
    std::vector<uint8_t> bytes(256);
    std::vector<uint32_t> off(257);
    for (int i = 0; i < 256; ++i) {
        bytes[size_t(i)] = uint8_t(i);
        off[size_t(i)] = uint32_t(i);
    }
    off[256] = 256;
    bfront_set_vocab(f, bytes.data(), off.data(), 256);
    bfront_set_lazy(f, 1);
    bfront_start(f);
    const int port = bfront_port(f);
    std::mutex mu;
    std::vector<int64_t> streams;
    std::atomic<bool> done{false};
    std::atomic<int> finished{0}, plain{0};

    std::thread dispatcher([&] {
        while (true) {
            int stopped = 0;
            void* ev = bfront_next_event(f, 50, &stopped);
            if (!ev) {
                if (stopped) return;
                continue;
            }
            int32_t kind;
            int64_t conn;
            uint32_t lens[5];
            memcpy(&kind, ev, 4);
            memcpy(&conn, static_cast<char*>(ev) + 4, 8);
            memcpy(lens, static_cast<char*>(ev) + 12, 20);
            std::string target(static_cast<char*>(ev) + 32 + lens[0], lens[1]);
            bfront_free(ev);
            if (kind != 1) continue;
            if (target == "/stream") {
                const uint8_t stops[] = {1, 0, 0, 0, 3, 0, 0, 0, 'E', 'N', 'D'};
                int64_t s = bfront_stream_open(f, conn, "{\"choices\": [{\"index\": 0, ", 1, stops, "data: {}\n\n", 0);
                if (s > 0) {
                    bfront_stream_begin(f, s, "content-type: text/event-stream\r\n");
                    std::lock_guard<std::mutex> lk(mu);
                    streams.push_back(s);
                }
            } else {
                bfront_respond(f, conn, 200, "content-type: text/plain\r\n", reinterpret_cast<const uint8_t*>("hello"), 5);
                plain++;
            }
        }
    });
    std::thread producer([&] {
        for (int step = 0; step < 400 && !done.load(); ++step) {
            std::vector<int64_t> cur;
            {
                std::lock_guard<std::mutex> lk(mu);
                cur = streams;
            }
            for (int64_t s : cur) bfront_stream_push(f, s, 97 + step % 26);
            bfront_kick(f);
            std::this_thread::sleep_for(std::chrono::microseconds(300));
        }
        std::lock_guard<std::mutex> lk(mu);
        for (int64_t s : streams) {
            bfront_stream_finish(f, s, "length", nullptr);
            finished++;
        }
        streams.clear();
    });
    std::vector<std::thread> clients;
    for (int c = 0; c < 8; ++c) {
        clients.emplace_back([&, c] {
            int fd = connect_to(port);
            if (fd < 0) return;
            const char* plain_req = "GET /x HTTP/1.1\r\nHost: a\r\n\r\n";
            const char* stream_req = "GET /stream HTTP/1.1\r\nHost: a\r\nConnection: close\r\n\r\n";
            char buf[8192];
            ssize_t w = write(fd, plain_req, strlen(plain_req));
            (void)w;
            ssize_t n = read(fd, buf, sizeof buf);
            (void)n;
            w = write(fd, stream_req, strlen(stream_req));
            (void)w;
            int reads = 0;
            while ((n = read(fd, buf, sizeof buf)) > 0) {
                if (c == 3 && ++reads == 5) break;          // this client leaves in mid-stream
            }
            close(fd);
        });
    }
    for (auto& t : clients) t.join();
    done.store(true);
    producer.join();
    int dangling = connect_to(port);                        // open while the front shuts down
    uint64_t st[8];
    bfront_stats(f, st);
    bfront_stop(f);
    dispatcher.join();
    bfront_destroy(f);
    if (dangling >= 0) close(dangling);
    std::printf("tsan driver ok: %d plain, %d streams finished, %llu tokens, %llu events\n", plain.load(), finished.load(),
                static_cast<unsigned long long>(st[2]), static_cast<unsigned long long>(st[3]));
    return plain.load() == 8 && finished.load() >= 7 ? 0 : 1;
}
