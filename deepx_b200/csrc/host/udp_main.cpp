// deepx-op-b200: the executor process.  Listens for deepxIR lines on UDP (default port 9090,
// the port of executor/op-cuda/src/client/main.cpp:27), runs each line and sends the reply
// datagram to the sender, as the reference's udpserver + main loop do
// (executor/deepxcore/src/client/udpserver.cpp:20-65, main.cpp:47-102).  Differences: a 64 KiB
// receive buffer instead of 1 KiB, no busy-polling queue between two threads (receive, run and
// reply happen on one thread, so the reply always goes to the sender of THAT line), and every
// exception becomes an error reply instead of ending the process.
//
// Environment: DEEPX_PORT (9090), DEEPX_DEVICE (0), DEEPX_POOL_BYTES (0 = unlimited),
// DEEPX_IR_LOG (1|true echoes each op), DEEPX_OP_TABLE (path to write the markdown op table),
// DEEPX_FUSE (0 turns the chain-fusion pass over multi-line datagrams off).  SIGUSR1 prints a
// counters line (ops run, tensors, pool bytes, fused chains); the same line is printed at exit.
#include <arpa/inet.h>
#include <sys/socket.h>
#include <unistd.h>

#include <csignal>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>

#include "core.hpp"

static volatile sig_atomic_t g_stop = 0, g_report = 0;
static void on_signal(int) { g_stop = 1; }
static void on_usr1(int) { g_report = 1; }

static void report(dxh::Executor &ex) {
    size_t st[4];
    dx_pool_stats(ex.mem().pool(), st);
    const dxh::FusionStats &f = ex.fusion_stats();
    std::cout << "deepx-op-b200: " << ex.ops_run() << " ops run, " << ex.mem().tensor_count() << " tensors, pool in use " << st[0]
              << " bytes, high-water " << st[2] << " bytes, " << st[3] << " driver allocations; fused chains: " << f.rmsnorm_groups
              << " rmsnorm, " << f.softmax_groups << " softmax, " << f.lines_absorbed << " IR lines absorbed" << std::endl;
}

int main() {
    using namespace dxh;
    const char *env;
    const int port = (env = std::getenv("DEEPX_PORT")) ? std::atoi(env) : 9090;
    const int device = (env = std::getenv("DEEPX_DEVICE")) ? std::atoi(env) : 0;
    const size_t limit = (env = std::getenv("DEEPX_POOL_BYTES")) ? std::strtoull(env, nullptr, 10) : 0;
    std::unique_ptr<Executor> ex;
    try {
        ex = std::make_unique<Executor>(device, limit);
    } catch (const std::exception &e) {
        std::cerr << "deepx-op-b200: " << e.what() << std::endl;
        return 1;
    }
    env = std::getenv("DEEPX_IR_LOG");
    ex->ir_log = env && (std::strcmp(env, "1") == 0 || strcasecmp(env, "true") == 0);
    if ((env = std::getenv("DEEPX_FUSE"))) ex->fuse = std::strcmp(env, "0") != 0;
    if ((env = std::getenv("DEEPX_OP_TABLE"))) {
        std::ofstream md(env);
        if (md.is_open()) md << ex->factory().print_markdown("op-b200");
    }

    const int fd = socket(AF_INET, SOCK_DGRAM, 0);
    if (fd < 0) { perror("socket creation failed"); return 1; }
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_addr.s_addr = INADDR_ANY;
    addr.sin_port = htons(uint16_t(port));
    if (bind(fd, reinterpret_cast<sockaddr *>(&addr), sizeof(addr)) < 0) { perror("bind failed"); close(fd); return 1; }
    timeval tv{0, 200000};  // wake up five times a second to notice SIGINT/SIGTERM
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    std::signal(SIGINT, on_signal);
    std::signal(SIGTERM, on_signal);
    std::signal(SIGUSR1, on_usr1);  // prints the counters line
    std::cout << "deepx-op-b200 listening on udp " << port << ", device " << device << ", " << ex->factory().size() << " ops" << std::endl;

    std::vector<char> buf(65536);
    while (!g_stop) {
        sockaddr_in cli{};
        socklen_t len = sizeof(cli);
        const ssize_t n = recvfrom(fd, buf.data(), buf.size() - 1, 0, reinterpret_cast<sockaddr *>(&cli), &len);
        if (g_report) {
            g_report = 0;
            report(*ex);
        }
        if (n <= 0) continue;
        buf[size_t(n)] = 0;
        // one reply datagram per IR line, in order; a datagram of several lines is a program
        // (chains of single ops inside it may run fused)
        for (const OpResp &r : ex->run_program(std::string(buf.data(), size_t(n)))) {
            const std::string reply = r.to_string();
            sendto(fd, reply.data(), reply.size(), 0, reinterpret_cast<sockaddr *>(&cli), len);
        }
    }
    report(*ex);
    close(fd);
    return 0;
}
