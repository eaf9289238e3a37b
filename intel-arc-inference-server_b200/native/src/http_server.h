// Minimal HTTP/1.1 server for the OpenAI-compatible API: request intake with a bounded FIFO,
// plain responses, and server-sent-event streams over chunked transfer encoding.
//
// The reference serves through cpp-httplib with a FIFO of depth 4 (a fifth waiting request gets
// 503), a role frame first on streams, "data: [DONE]" last, and cancels generation when the
// client goes away (src/server/server.cc:176-184, :717-769; server.h:28-35).  This transport
// keeps those rules and nothing else: connection threads parse a request and park it in the
// queue; the serving loop (which owns the engine) takes requests with next(), answers with
// respond() or begin_stream() / send_event() / end_stream(), and polls cancelled().
#pragma once
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace b2host {

struct HttpRequest {
  uint64_t id = 0;
  std::string method, path, body;
  std::map<std::string, std::string> headers;
};

class HttpServer {
 public:
  HttpServer(const std::string& host, int port, int max_waiting = 4) : max_waiting_(max_waiting) {
    fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd_ < 0) throw std::runtime_error("socket() failed");
    int one = 1;
    setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1) addr.sin_addr.s_addr = htonl(INADDR_ANY);
    if (::bind(fd_, (sockaddr*)&addr, sizeof addr) != 0) {
      ::close(fd_);
      throw std::runtime_error("bind() failed: " + std::string(strerror(errno)));
    }
    socklen_t len = sizeof addr;
    getsockname(fd_, (sockaddr*)&addr, &len);
    port_ = ntohs(addr.sin_port);
    if (::listen(fd_, 64) != 0) throw std::runtime_error("listen() failed");
    acceptor_ = std::thread([this] { accept_loop(); });
  }
  ~HttpServer() { stop(); }
  int port() const { return port_; }

  void stop() {
    if (stopping_.exchange(true)) return;
    ::shutdown(fd_, SHUT_RDWR);
    ::close(fd_);
    cv_.notify_all();
    if (acceptor_.joinable()) acceptor_.join();
    {
      std::lock_guard<std::mutex> g(mu_);
      for (auto& kv : conns_) ::shutdown(kv.second->fd, SHUT_RDWR);
    }
    // connection threads are detached; they leave within one poll interval once stopping_ is set
    for (int i = 0; i < 200 && active_.load() > 0; ++i) std::this_thread::sleep_for(std::chrono::milliseconds(10));
  }

  // Next queued request, or id 0 after timeout_ms.  `in_flight` requests (taken, not yet answered)
  // count against nothing: only WAITING requests are bounded.
  HttpRequest next(int timeout_ms) {
    std::unique_lock<std::mutex> g(mu_);
    cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), [&] { return !queue_.empty() || stopping_; });
    if (queue_.empty()) return HttpRequest();
    HttpRequest r = std::move(queue_.front());
    queue_.pop_front();
    return r;
  }
  int active() const { return active_.load(); }   // connection threads alive
  int waiting() {
    std::lock_guard<std::mutex> g(mu_);
    return (int)queue_.size();
  }
  bool cancelled(uint64_t id) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = conns_.find(id);
    return it == conns_.end() || it->second->gone;
  }

  bool respond(uint64_t id, int status, const std::string& content_type, const std::string& body) {
    auto c = conn(id);
    if (!c) return false;
    std::string h = "HTTP/1.1 " + std::to_string(status) + " " + reason(status) + "\r\nContent-Type: " + content_type +
                    "\r\nContent-Length: " + std::to_string(body.size()) + "\r\nConnection: close\r\n\r\n";
    const bool ok = write_all(c, h + body);
    finish(id);
    return ok;
  }
  // Drops a request that will get no answer (its client went away before a slot was granted): the connection
  // thread stops watching the socket and closes it.
  void close(uint64_t id) { finish(id); }
  bool begin_stream(uint64_t id) {
    auto c = conn(id);
    if (!c) return false;
    return write_all(c,
                     "HTTP/1.1 200 OK\r\nContent-Type: text/event-stream\r\nCache-Control: no-cache\r\n"
                     "Transfer-Encoding: chunked\r\nConnection: close\r\n\r\n");
  }
  bool send_event(uint64_t id, const std::string& data) {
    auto c = conn(id);
    if (!c) return false;
    const std::string payload = "data: " + data + "\n\n";
    char hex[32];
    snprintf(hex, sizeof hex, "%zx\r\n", payload.size());
    return write_all(c, std::string(hex) + payload + "\r\n");
  }
  bool end_stream(uint64_t id) {
    const bool ok = send_event(id, "[DONE]");
    auto c = conn(id);
    if (c) write_all(c, "0\r\n\r\n");
    finish(id);
    return ok;
  }

 private:
  struct Conn {
    int fd = -1;
    std::atomic<bool> gone{false};
    std::mutex wmu;
    std::condition_variable done_cv;
    bool done = false;
  };

  static const char* reason(int s) {
    switch (s) {
      case 200: return "OK";
      case 400: return "Bad Request";
      case 404: return "Not Found";
      case 405: return "Method Not Allowed";
      case 413: return "Payload Too Large";
      case 500: return "Internal Server Error";
      case 503: return "Service Unavailable";
    }
    return "Status";
  }
  std::shared_ptr<Conn> conn(uint64_t id) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = conns_.find(id);
    return it == conns_.end() ? nullptr : it->second;
  }
  bool write_all(const std::shared_ptr<Conn>& c, const std::string& data) {
    std::lock_guard<std::mutex> g(c->wmu);
    if (c->gone) return false;
    size_t off = 0;
    while (off < data.size()) {
      const ssize_t n = ::send(c->fd, data.data() + off, data.size() - off, MSG_NOSIGNAL);
      if (n <= 0) {
        c->gone = true;
        return false;
      }
      off += (size_t)n;
    }
    return true;
  }
  void finish(uint64_t id) {
    std::shared_ptr<Conn> c;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = conns_.find(id);
      if (it == conns_.end()) return;
      c = it->second;
    }
    std::lock_guard<std::mutex> g(c->wmu);
    c->done = true;
    c->done_cv.notify_all();
  }

  void accept_loop() {
    while (!stopping_) {
      sockaddr_in peer{};
      socklen_t len = sizeof peer;
      const int cfd = ::accept(fd_, (sockaddr*)&peer, &len);
      if (cfd < 0) {
        if (stopping_) return;
        continue;
      }
      int one = 1;
      setsockopt(cfd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
      // a client that stops reading must not hold the serving thread: a send that cannot make progress for this
      // long fails, and write_all marks the connection gone (its request is then cancelled like a hang-up)
      timeval snd{kSendTimeoutSec, 0};
      setsockopt(cfd, SOL_SOCKET, SO_SNDTIMEO, &snd, sizeof snd);
      ++active_;
      std::thread([this, cfd] {
        serve(cfd);
        --active_;
      }).detach();
    }
  }

  static bool read_request(int fd, HttpRequest& r, int* err_status) {
    std::string buf;
    size_t header_end = std::string::npos;
    char tmp[8192];
    while (header_end == std::string::npos) {
      const ssize_t n = ::recv(fd, tmp, sizeof tmp, 0);
      if (n <= 0) return false;
      buf.append(tmp, (size_t)n);
      header_end = buf.find("\r\n\r\n");
      if (buf.size() > (1u << 20) && header_end == std::string::npos) { *err_status = 413; return false; }
    }
    const std::string head = buf.substr(0, header_end);
    size_t line_end = head.find("\r\n");
    const std::string req_line = head.substr(0, line_end);
    const size_t s1 = req_line.find(' '), s2 = req_line.rfind(' ');
    if (s1 == std::string::npos || s2 == s1) { *err_status = 400; return false; }
    r.method = req_line.substr(0, s1);
    r.path = req_line.substr(s1 + 1, s2 - s1 - 1);
    const size_t qm = r.path.find('?');
    if (qm != std::string::npos) r.path.erase(qm);
    size_t pos = line_end == std::string::npos ? head.size() : line_end + 2;
    while (pos < head.size()) {
      size_t e = head.find("\r\n", pos);
      if (e == std::string::npos) e = head.size();
      const std::string line = head.substr(pos, e - pos);
      const size_t colon = line.find(':');
      if (colon != std::string::npos) {
        std::string k = line.substr(0, colon), v = line.substr(colon + 1);
        for (auto& ch : k) ch = (char)tolower((unsigned char)ch);
        while (!v.empty() && v.front() == ' ') v.erase(0, 1);
        r.headers[k] = v;
      }
      pos = e + 2;
    }
    size_t want = 0;
    auto cl = r.headers.find("content-length");
    if (cl != r.headers.end()) want = (size_t)strtoull(cl->second.c_str(), nullptr, 10);
    if (want > (256u << 20)) { *err_status = 413; return false; }
    r.body = buf.substr(header_end + 4);
    while (r.body.size() < want) {
      const ssize_t n = ::recv(fd, tmp, sizeof tmp, 0);
      if (n <= 0) return false;
      r.body.append(tmp, (size_t)n);
    }
    r.body.resize(want);
    return true;
  }

  void serve(int cfd) {
    HttpRequest r;
    int err = 0;
    auto c = std::make_shared<Conn>();
    c->fd = cfd;
    if (!read_request(cfd, r, &err)) {
      if (err) {
        const std::string body = "{\"error\":{\"message\":\"bad request\",\"type\":\"invalid_request_error\"}}";
        const std::string h = "HTTP/1.1 " + std::to_string(err) + " " + reason(err) +
                              "\r\nContent-Type: application/json\r\nContent-Length: " + std::to_string(body.size()) +
                              "\r\nConnection: close\r\n\r\n" + body;
        ::send(cfd, h.data(), h.size(), MSG_NOSIGNAL);
      }
      ::close(cfd);
      return;
    }
    {
      std::unique_lock<std::mutex> g(mu_);
      if ((int)queue_.size() >= max_waiting_) {
        g.unlock();
        const std::string body =
            "{\"error\":{\"message\":\"server is busy: too many requests waiting\",\"type\":\"server_error\",\"code\":503}}";
        const std::string h = "HTTP/1.1 503 Service Unavailable\r\nContent-Type: application/json\r\nRetry-After: 1\r\n"
                              "Content-Length: " + std::to_string(body.size()) + "\r\nConnection: close\r\n\r\n" + body;
        ::send(cfd, h.data(), h.size(), MSG_NOSIGNAL);
        ::close(cfd);
        return;
      }
      r.id = ++next_id_;
      conns_[r.id] = c;
      queue_.push_back(r);
    }
    cv_.notify_one();
    // watch the socket until the serving loop is done with it; a hang-up marks the request cancelled
    for (;;) {
      {
        std::unique_lock<std::mutex> g(c->wmu);
        if (c->done_cv.wait_for(g, std::chrono::milliseconds(50), [&] { return c->done; })) break;
      }
      if (stopping_) break;
      pollfd p{cfd, POLLIN | POLLRDHUP, 0};
      if (::poll(&p, 1, 0) > 0 && (p.revents & (POLLRDHUP | POLLHUP | POLLERR))) {
        c->gone = true;
      } else if (p.revents & POLLIN) {
        char tmp[256];
        if (::recv(cfd, tmp, sizeof tmp, MSG_DONTWAIT) == 0) c->gone = true;
      }
    }
    {
      std::lock_guard<std::mutex> g(mu_);
      conns_.erase(r.id);
    }
    ::shutdown(cfd, SHUT_RDWR);
    ::close(cfd);
  }

  static constexpr int kSendTimeoutSec = 5;
  int fd_ = -1, port_ = 0, max_waiting_;
  std::atomic<bool> stopping_{false};
  std::thread acceptor_;
  std::atomic<int> active_{0};
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<HttpRequest> queue_;
  std::map<uint64_t, std::shared_ptr<Conn>> conns_;
  uint64_t next_id_ = 0;
};

}  // namespace b2host
