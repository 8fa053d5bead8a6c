// part_workers.h -- the rounds of several sumcheck contexts at the same time.
//
// A statement proved in parts (one context per part: the lookups of a LogUp-GKR layer, the groups of
// terms of a wide statement) needs every part's sums of a round before the round's message can be
// sent.  sc_round launches and waits, so calling it part after part would add the parts' latencies;
// here part 0 runs on the calling thread and every other part on a thread of its own, which lives
// for the length of one proof and spins between rounds (a round lasts microseconds).
#pragma once
#include <atomic>
#include <cstdint>
#include <memory>
#include <thread>
#include <vector>

#include "../../include/sumcheck_b200.h"

namespace sc {

class PartWorkers {
  public:
    explicit PartWorkers(const std::vector<sc_ctx *> &ctxs) : ctxs_(ctxs) {
        for (size_t k = 1; k < ctxs.size(); k++) {
            workers_.emplace_back(new Worker());
            Worker *w = workers_.back().get();
            w->ctx = ctxs[k];
            w->thread = std::thread([w] {
                int seen = 0;
                for (;;) {
                    int cmd;
                    while ((cmd = w->cmd.load(std::memory_order_acquire)) == seen) pause();
                    if (cmd < 0) return;
                    seen = cmd;
                    w->rc = sc_round(w->ctx, w->sums);
                    w->done.store(cmd, std::memory_order_release);
                }
            });
        }
    }
    ~PartWorkers() {
        for (auto &w : workers_) { w->cmd.store(-1, std::memory_order_release); w->thread.join(); }
    }
    PartWorkers(const PartWorkers &) = delete;
    PartWorkers &operator=(const PartWorkers &) = delete;

    // One round on every context; SUMS gets the words of part 0, PART(k) those of part k >= 1 afterwards.
    // Returns the first error code.
    int round(uint32_t *sums) {
        ++seq_;
        for (auto &w : workers_) w->cmd.store(seq_, std::memory_order_release);
        int rc = sc_round(ctxs_[0], sums);
        for (auto &w : workers_) {
            while (w->done.load(std::memory_order_acquire) != seq_) pause();
            if (!rc) rc = w->rc;
        }
        return rc;
    }
    const uint32_t *part(size_t k) const { return workers_[k - 1]->sums; }

  private:
    struct Worker {
        std::thread thread;
        std::atomic<int> cmd{0}, done{0};
        int rc = 0;
        sc_ctx *ctx = nullptr;
        uint32_t sums[SC_MAX_POINTS * 8];
    };
    static void pause() {
#if defined(__x86_64__) || defined(__i386__)
        __builtin_ia32_pause();
#else
        std::this_thread::yield();
#endif
    }
    std::vector<sc_ctx *> ctxs_;
    std::vector<std::unique_ptr<Worker>> workers_;
    int seq_ = 0;
};

}  // namespace sc
