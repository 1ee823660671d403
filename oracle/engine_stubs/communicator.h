// Test infrastructure, not product code.
//
// Single-process stand-in for the reference's UCX communicator (src/engine/communicator.h; UCX is
// not installed here), shadowing it in the include mirror so that the reference's engine sources
// compile unchanged.  Only what src/engine/{notifier,channel_manager}.cc call is declared.  With
// one process nothing ever sends: the GPU server never instantiates the notifier or the channel
// managers (src/server/gpu/server.cc:114-121), so every transfer entry point throws.
#pragma once
#include "../base/setup.h"

#include "threadpool.h"

struct communicator_t {
    int get_this_rank() const { return 0; }
    int get_world_size() const { return 1; }
    int num_channels(int) const { return 1; }
    void barrier() {}

    void start_listen_notify(uint64_t, std::function<bool(vector<uint8_t>)>, bool = false) {}
    void stop_listen_notify() {}
    void notify(int, void const*, uint64_t) { none(); }
    void send(int, int, void const*, uint64_t) { none(); }
    void recv(int, int, void*, uint64_t) { none(); }

private:
    [[noreturn]] static void none()
    {
        throw std::runtime_error("communicator stub: a single process has no peer to talk to");
    }
};
