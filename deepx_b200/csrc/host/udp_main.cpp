// deepx-op-b200: the executor process.  Listens for deepxIR lines on UDP (default port 9090,
// the port of executor/op-cuda/src/client/main.cpp:27), runs each line and sends the reply
// datagram to the sender, as the reference's udpserver + main loop do
// (executor/deepxcore/src/client/udpserver.cpp:20-65, main.cpp:47-102).  Differences: a 64 KiB
// receive buffer instead of 1 KiB, no busy-polling queue between two threads (receive, run and
// reply happen on one thread, so the reply always goes to the sender of THAT line), every
// exception becomes an error reply instead of ending the process, and the socket listens on the
// loopback address unless DEEPX_BIND says otherwise (IR lines name files to read and write).
//
// Several GPUs (DEEPX_DEVICES=0,1,2,3): the process forks one worker per device before anything
// touches CUDA.  Each worker is an executor that is one rank of the world (dx_exec_set_shard): large
// tensors are partitioned by rows over the workers, reductions over axis 0 are combined over NVLink
// peer memory.  The front process hands every datagram to all workers, waits for all their replies and
// answers the sender with rank 0's reply per line — or with the first error any rank reported.  The
// scheduler and the front ends see one executor on one port, as before.
//
// Environment: DEEPX_PORT (9090), DEEPX_BIND (127.0.0.1; 0.0.0.0 or an address of this host to accept
// remote senders), DEEPX_DEVICE (0) or DEEPX_DEVICES (comma-separated list), DEEPX_SHARD_MIN_BYTES
// (1048576: tensors at least this large are partitioned when there are several devices), DEEPX_POOL_BYTES
// (0 = unlimited, per device), DEEPX_IR_LOG (1|true echoes each op), DEEPX_OP_TABLE (path to write the
// markdown op table), DEEPX_FUSE (0 turns the chain-fusion pass over multi-line datagrams off).
// SIGUSR1 prints a counters line (ops run, tensors, pool bytes, fused chains); the same line is printed
// at exit.
#include <arpa/inet.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cerrno>
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

static void report(dxh::Executor &ex, int rank, int world) {
    size_t st[4];
    dx_pool_stats(ex.mem().pool(), st);
    const dxh::FusionStats &f = ex.fusion_stats();
    std::cout << "deepx-op-b200";
    if (world > 1) std::cout << "[" << rank << "/" << world << "]";
    std::cout << ": " << ex.ops_run() << " ops run, " << ex.mem().tensor_count() << " tensors, pool in use " << st[0]
              << " bytes, high-water " << st[2] << " bytes, " << st[3] << " driver allocations; fused chains: " << f.rmsnorm_groups
              << " rmsnorm, " << f.softmax_groups << " softmax, " << f.lines_absorbed << " IR lines absorbed" << std::endl;
}

static std::unique_ptr<dxh::Executor> make_executor(int device, size_t limit) {
    auto ex = std::make_unique<dxh::Executor>(device, limit);
    const char *env = std::getenv("DEEPX_IR_LOG");
    ex->ir_log = env && (std::strcmp(env, "1") == 0 || strcasecmp(env, "true") == 0);
    if ((env = std::getenv("DEEPX_FUSE"))) ex->fuse = std::strcmp(env, "0") != 0;
    return ex;
}

static std::string join_replies(const std::vector<dxh::OpResp> &rs) {
    std::string all;
    for (size_t i = 0; i < rs.size(); ++i) {
        if (i) all += "\n";
        all += rs[i].to_string();
    }
    return all;
}

// ---- one worker of a multi-device executor: talks to the front process over a socket pair --------------
static bool send_msg(int fd, const std::string &m) { return send(fd, m.data(), m.size(), MSG_NOSIGNAL) == ssize_t(m.size()); }
static bool recv_msg(int fd, std::string &m) {
    std::vector<char> buf(1 << 20);
    ssize_t n;
    do n = recv(fd, buf.data(), buf.size(), 0);
    while (n < 0 && errno == EINTR);  // a signal (SIGUSR1 asks for the counters line) is not the end of the conversation
    if (n < 0) return false;
    m.assign(buf.data(), size_t(n));
    return true;
}

static int worker_main(int fd, int rank, int world, int device, size_t limit, size_t min_bytes) {
    std::signal(SIGINT, SIG_IGN);  // the front process decides when the workers stop
    std::unique_ptr<dxh::Executor> ex;
    dx_comm *comm = nullptr;
    std::string msg;
    try {
        ex = make_executor(device, limit);
        comm = dx_comm_create(rank, world, device);
        unsigned char handle[64];
        if (!comm || dx_comm_handle(comm, handle) != DX_OK) throw std::runtime_error(dx_last_error());
        if (!send_msg(fd, "H" + std::string(reinterpret_cast<char *>(handle), 64))) throw std::runtime_error("front process is gone");
        if (!recv_msg(fd, msg) || msg.size() != size_t(64 * world)) throw std::runtime_error("bad handle table from the front process");
        if (dx_comm_connect(comm, reinterpret_cast<const unsigned char *>(msg.data())) != DX_OK) throw std::runtime_error(dx_last_error());
        ex->set_shard(rank, world, min_bytes, comm);
        send_msg(fd, "R");
    } catch (const std::exception &e) {
        send_msg(fd, std::string("E") + e.what());
        return 1;
    }
    std::signal(SIGUSR1, on_usr1);
    while (recv_msg(fd, msg) && !msg.empty() && msg != "\x04") {
        if (g_report) {
            g_report = 0;
            report(*ex, rank, world);
        }
        if (!send_msg(fd, join_replies(ex->run_program(msg)))) break;
    }
    report(*ex, rank, world);
    ex.reset();
    dx_comm_destroy(comm);
    return 0;
}

int main() {
    using namespace dxh;
    const char *env;
    const int port = (env = std::getenv("DEEPX_PORT")) ? std::atoi(env) : 9090;
    const std::string bind_to = (env = std::getenv("DEEPX_BIND")) ? env : "127.0.0.1";
    const size_t limit = (env = std::getenv("DEEPX_POOL_BYTES")) ? std::strtoull(env, nullptr, 10) : 0;
    const size_t min_bytes = (env = std::getenv("DEEPX_SHARD_MIN_BYTES")) ? std::strtoull(env, nullptr, 10) : (size_t(1) << 20);
    std::vector<int> devices;
    if ((env = std::getenv("DEEPX_DEVICES")) && *env) {
        std::istringstream ds(env);
        std::string item;
        while (std::getline(ds, item, ','))
            if (!item.empty()) devices.push_back(std::atoi(item.c_str()));
    }
    if (devices.empty()) devices.push_back((env = std::getenv("DEEPX_DEVICE")) ? std::atoi(env) : 0);
    const int world = int(devices.size());
    if (world > 16) { std::cerr << "deepx-op-b200: at most 16 devices" << std::endl; return 1; }

    // several devices: fork the workers first, while this process has not touched CUDA
    std::vector<int> fds;
    std::vector<pid_t> pids;
    if (world > 1) {
        for (int r = 0; r < world; ++r) {
            int sv[2];
            if (socketpair(AF_UNIX, SOCK_SEQPACKET, 0, sv) != 0) { perror("socketpair"); return 1; }
            const pid_t pid = fork();
            if (pid < 0) { perror("fork"); return 1; }
            if (pid == 0) {
                close(sv[0]);
                for (int f : fds) close(f);
                _exit(worker_main(sv[1], r, world, devices[size_t(r)], limit, min_bytes));
            }
            close(sv[1]);
            fds.push_back(sv[0]);
            pids.push_back(pid);
        }
        // the mailbox handles of all workers, handed back to each of them
        std::string table(size_t(64 * world), '\0'), msg;
        bool ok = true;
        for (int r = 0; r < world && ok; ++r) {
            ok = recv_msg(fds[size_t(r)], msg) && msg.size() == 65 && msg[0] == 'H';
            if (ok) table.replace(size_t(64 * r), 64, msg, 1, 64);
            else std::cerr << "deepx-op-b200: worker " << r << " (device " << devices[size_t(r)] << ") failed to start: " << (msg.size() > 1 ? msg.substr(1) : "no answer") << std::endl;
        }
        for (int r = 0; r < world && ok; ++r) ok = send_msg(fds[size_t(r)], table);
        for (int r = 0; r < world && ok; ++r) {
            ok = recv_msg(fds[size_t(r)], msg) && msg == "R";
            if (!ok) std::cerr << "deepx-op-b200: worker " << r << " could not reach its peers: " << (msg.size() > 1 ? msg.substr(1) : "no answer") << std::endl;
        }
        if (!ok) {
            for (int f : fds) close(f);
            for (pid_t p : pids) waitpid(p, nullptr, 0);
            return 1;
        }
    }

    std::unique_ptr<Executor> ex;
    if (world == 1) {
        try {
            ex = make_executor(devices[0], limit);
        } catch (const std::exception &e) {
            std::cerr << "deepx-op-b200: " << e.what() << std::endl;
            return 1;
        }
    }
    TfFactory table;  // the op table does not depend on a device
    register_all(table);
    register_fused(table);
    if ((env = std::getenv("DEEPX_OP_TABLE"))) {
        std::ofstream md(env);
        if (md.is_open()) md << table.print_markdown("op-b200");
    }

    const int fd = socket(AF_INET, SOCK_DGRAM, 0);
    if (fd < 0) { perror("socket creation failed"); return 1; }
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    if (inet_pton(AF_INET, bind_to.c_str(), &addr.sin_addr) != 1) { std::cerr << "deepx-op-b200: DEEPX_BIND is not an IPv4 address: " << bind_to << std::endl; return 1; }
    addr.sin_port = htons(uint16_t(port));
    if (bind(fd, reinterpret_cast<sockaddr *>(&addr), sizeof(addr)) < 0) { perror("bind failed"); close(fd); return 1; }
    timeval tv{0, 200000};  // wake up five times a second to notice SIGINT/SIGTERM
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    std::signal(SIGINT, on_signal);
    std::signal(SIGTERM, on_signal);
    std::signal(SIGUSR1, on_usr1);  // prints the counters line
    std::cout << "deepx-op-b200 listening on udp " << bind_to << ":" << port << ", device";
    for (int r = 0; r < world; ++r) std::cout << (r ? "," : (world > 1 ? "s " : " ")) << devices[size_t(r)];
    std::cout << ", " << table.size() << " ops" << std::endl;

    std::vector<char> buf(65536);
    bool workers_ok = true;
    while (!g_stop && workers_ok) {
        sockaddr_in cli{};
        socklen_t len = sizeof(cli);
        const ssize_t n = recvfrom(fd, buf.data(), buf.size() - 1, 0, reinterpret_cast<sockaddr *>(&cli), &len);
        if (g_report) {
            g_report = 0;
            if (ex) report(*ex, 0, 1);
            for (pid_t p : pids) kill(p, SIGUSR1);  // each worker prints its own line with its next datagram
        }
        if (n <= 0) continue;
        buf[size_t(n)] = 0;
        const std::string program(buf.data(), size_t(n));
        // one reply datagram per IR line, in order; a datagram of several lines is a program
        // (chains of single ops inside it may run fused)
        if (ex) {
            for (const OpResp &r : ex->run_program(program)) {
                const std::string reply = r.to_string();
                sendto(fd, reply.data(), reply.size(), 0, reinterpret_cast<sockaddr *>(&cli), len);
            }
            continue;
        }
        if (program.find_first_not_of(" \t\r\n") == std::string::npos) continue;
        for (int r = 0; r < world && workers_ok; ++r) workers_ok = send_msg(fds[size_t(r)], program);
        std::vector<std::vector<std::string>> replies(static_cast<size_t>(world));
        for (int r = 0; r < world && workers_ok; ++r) {
            std::string all;
            workers_ok = recv_msg(fds[size_t(r)], all);
            std::istringstream ls(all);
            std::string line;
            while (std::getline(ls, line)) replies[size_t(r)].push_back(line);
        }
        if (!workers_ok) {
            const std::string reply = "0 error// a worker of this executor is gone";
            sendto(fd, reply.data(), reply.size(), 0, reinterpret_cast<sockaddr *>(&cli), len);
            break;
        }
        for (size_t i = 0; i < replies[0].size(); ++i) {
            std::string reply = replies[0][i];
            for (int r = 0; r < world; ++r) {  // the first rank that reported an error speaks for the line
                const std::string &cand = i < replies[size_t(r)].size() ? replies[size_t(r)][i] : reply;
                const size_t sp = cand.find(' ');
                if (sp != std::string::npos && cand.compare(sp + 1, 5, "error") == 0) { reply = cand; break; }
            }
            sendto(fd, reply.data(), reply.size(), 0, reinterpret_cast<sockaddr *>(&cli), len);
        }
    }
    if (ex) report(*ex, 0, 1);
    for (int f : fds) {
        send_msg(f, "\x04");
        close(f);
    }
    for (pid_t p : pids) waitpid(p, nullptr, 0);
    close(fd);
    return workers_ok ? 0 : 1;
}
