// part_workers.h -- the rounds of several sumcheck contexts at the same time.
//
// A statement proved in parts (one context per part: the lookups of a LogUp-GKR layer, the groups of
// terms of a wide statement) needs every part's sums of a round before the round's message can be
// sent.  sc_round launches and waits, so calling it part after part would add the parts' latencies;
// here part 0 runs on the calling thread and the other parts on helper threads that live for the
// length of one proof.  There are never more helpers than the host has spare cores (the parts are
// dealt out among them), a helper spins only briefly between rounds and then yields its core, and
// if no thread can be started the parts simply run one after the other on the calling thread.
#pragma once
#include <atomic>
#include <cstdint>
#include <memory>
#include <system_error>
#include <thread>
#include <vector>

#include "../../include/sumcheck_b200.h"

namespace sc {

class PartWorkers {
  public:
    explicit PartWorkers(const std::vector<sc_ctx *> &ctxs) : ctxs_(ctxs), sums_(ctxs.size()) {
        const size_t others = ctxs.size() > 1 ? ctxs.size() - 1 : 0;
        unsigned cores = std::thread::hardware_concurrency();
        if (cores == 0) cores = 2;
        size_t helpers = cores > 1 ? cores - 1 : 0;
        if (helpers > others) helpers = others;
        for (size_t w = 0; w < helpers; w++) {
            std::unique_ptr<Worker> wk(new Worker());
            for (size_t k = 1 + w; k < ctxs.size(); k += helpers) wk->parts.push_back(k);
            Worker *p = wk.get();
            try {
                p->thread = std::thread([this, p] { run(p); });
            } catch (const std::system_error &) {
                break;   // no more threads to be had: the parts not dealt out yet run on the calling thread
            }
            workers_.push_back(std::move(wk));
        }
        std::vector<bool> taken(ctxs.size(), false);
        for (auto &w : workers_) for (size_t k : w->parts) taken[k] = true;
        for (size_t k = 1; k < ctxs.size(); k++) if (!taken[k]) mine_.push_back(k);
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
        for (size_t k : mine_) { const int r = sc_round(ctxs_[k], sums_[k].w); if (!rc) rc = r; }
        for (auto &w : workers_) {
            unsigned spins = 0;
            while (w->done.load(std::memory_order_acquire) != seq_) pause(++spins);
            if (!rc) rc = w->rc;
        }
        return rc;
    }
    const uint32_t *part(size_t k) const { return sums_[k].w; }

  private:
    struct Sums { uint32_t w[SC_MAX_POINTS * 8]; };
    struct Worker {
        std::thread thread;
        std::atomic<int> cmd{0}, done{0};
        int rc = 0;
        std::vector<size_t> parts;
    };
    void run(Worker *w) {
        int seen = 0;
        for (;;) {
            int cmd;
            unsigned spins = 0;
            while ((cmd = w->cmd.load(std::memory_order_acquire)) == seen) pause(++spins);
            if (cmd < 0) return;
            seen = cmd;
            int rc = 0;
            for (size_t k : w->parts) { const int r = sc_round(ctxs_[k], sums_[k].w); if (!rc) rc = r; }
            w->rc = rc;
            w->done.store(cmd, std::memory_order_release);
        }
    }
    // a round lasts microseconds, so a short spin catches the next one; after that the core is given up
    static void pause(unsigned spins) {
        if (spins > 20000) { std::this_thread::yield(); return; }
#if defined(__x86_64__) || defined(__i386__)
        __builtin_ia32_pause();
#endif
    }
    std::vector<sc_ctx *> ctxs_;
    std::vector<Sums> sums_;
    std::vector<std::unique_ptr<Worker>> workers_;
    std::vector<size_t> mine_;
    int seq_ = 0;
};

}  // namespace sc
