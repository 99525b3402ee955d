// Unit test of the work-counter hand-out (tt-buda_b200/csrc/work_slots.hpp) against a fake completion backend:
// no GPU involved.  Exits 0 when every check holds; prints the failing check otherwise.
#include <cstdio>
#include <set>
#include <thread>
#include <vector>

#include "work_slots.hpp"

using buda::WorkSlotRing;

struct FakeBackend {
    bool running[64] = {};
    int waits = 0;
    bool busy(int slot) { return running[slot]; }
    void wait(int slot) { waits++; running[slot] = false; }
};

#define CHECK(cond)                                                      \
    do {                                                                 \
        if (!(cond)) {                                                   \
            std::printf("FAILED line %d: %s\n", __LINE__, #cond);        \
            return 1;                                                    \
        }                                                                \
    } while (0)

int main()
{
    {   // a busy slot is never handed out: 8 ordinary slots, launches that never finish
        WorkSlotRing<12, 4> ring;
        FakeBackend be;
        std::set<int> seen;
        for (int i = 0; i < 8; i++) {
            const int s = ring.acquire(be);
            CHECK(s >= 0 && s < 8 && !seen.count(s));
            seen.insert(s);
            be.running[s] = true;   // its launch is now in flight
            ring.release(s);
        }
        // all 8 in flight: the next request has to wait for one of them, never shares
        CHECK(be.waits == 0);
        const int s = ring.acquire(be);
        CHECK(s >= 0 && s < 8 && be.waits == 1 && !be.running[s]);
        be.running[s] = true;
        ring.release(s);
        // finished launches free their slots without waiting
        be.running[3] = be.running[5] = false;
        const int a = ring.acquire(be);
        be.running[a] = true;
        ring.release(a);
        const int b = ring.acquire(be);
        be.running[b] = true;
        ring.release(b);
        CHECK((a == 3 && b == 5) || (a == 5 && b == 3));
        CHECK(be.waits == 1);
    }
    {   // a slot in another thread's hands (acquired, launch not yet marked) is skipped even if its old launch is done
        WorkSlotRing<6, 2> ring;
        FakeBackend be;
        const int a = ring.acquire(be);
        const int b = ring.acquire(be);
        const int c = ring.acquire(be);
        const int d = ring.acquire(be);
        CHECK(a != b && a != c && a != d && b != c && b != d && c != d);
        CHECK(ring.acquire(be) == -1);   // four ordinary slots, all in hand
        ring.release(b);
        CHECK(ring.acquire(be) == b);
    }
    {   // capture slots: outside the ordinary range, never twice, refused when used up
        WorkSlotRing<12, 4> ring;
        std::set<int> seen;
        for (int i = 0; i < 4; i++) {
            const int s = ring.acquire_for_capture();
            CHECK(s >= 8 && s < 12 && !seen.count(s));
            seen.insert(s);
        }
        CHECK(ring.acquire_for_capture() == -1);
        FakeBackend be;
        for (int i = 0; i < 100; i++) {
            const int s = ring.acquire(be);
            CHECK(s >= 0 && s < 8);
            ring.release(s);
        }
    }
    {   // many threads: no two hold the same slot at once
        WorkSlotRing<40, 8> ring;
        struct Shared {
            std::mutex mu;
            bool held[40] = {};
            bool clash = false;
            bool busy(int) { return false; }
            void wait(int) {}
        } sh;
        std::vector<std::thread> ts;
        for (int t = 0; t < 8; t++)
            ts.emplace_back([&] {
                for (int i = 0; i < 20000; i++) {
                    const int s = ring.acquire(sh);
                    if (s < 0) continue;
                    {
                        std::lock_guard<std::mutex> l(sh.mu);
                        if (sh.held[s]) sh.clash = true;
                        sh.held[s] = true;
                    }
                    {
                        std::lock_guard<std::mutex> l(sh.mu);
                        sh.held[s] = false;
                    }
                    ring.release(s);
                }
            });
        for (auto &t : ts) t.join();
        CHECK(!sh.clash);
    }
    std::printf("ok\n");
    return 0;
}
