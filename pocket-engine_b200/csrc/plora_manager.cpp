// Adapter lifecycle around the registry, as the engine thread runs it (src/engine.rs:490-655): adapters are read
// and laid out on worker threads while the engine keeps serving; finished ones are registered and their callers
// answered from the engine thread; adapters loaded on demand are dropped least recently used first once more
// than max_cpu_loras are resident; an unloaded adapter that requests still use drains before it is freed.
// Everything except the worker's read runs on the caller's (engine) thread, like the registry itself.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <memory>
#include <cstring>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <vector>

#include "plora_internal.h"

extern "C" int plora_adapter_read(const plora_t* h, const char* name, const char* path, plora_adapter_t** out);

struct plora_manager {
    plora_t* h = nullptr;
    plora_slots_t* slots = nullptr;  // optional: forgotten adapters leave their GPU slots (src/sched.rs:569-585)
    int max_cpu_loras = 0;

    struct Prepared {  // src/engine.rs Prepared
        std::string name, path, error;
        plora_adapter_t* adapter = nullptr;
        int rc = PLORA_OK;
        bool on_demand = false;
    };
    struct Reply {
        bool done = false;
        int status = PLORA_OK;
        std::string text;
    };
    std::mutex mu;  // guards `prepared` and `live_workers` (the only state workers touch)
    std::condition_variable cv;
    std::deque<Prepared> prepared;
    int live_workers = 0;
    struct Worker {
        std::thread t;
        std::shared_ptr<std::atomic<bool>> done;
    };
    std::vector<Worker> workers;

    std::map<uint64_t, Reply> replies;
    uint64_t next_ticket = 1;
    std::map<std::string, std::vector<uint64_t>> loading;  // name -> tickets waiting for it
    std::set<uint32_t> on_demand;
    std::map<uint32_t, uint64_t> last_used;  // a logical clock, advanced on every touch
    uint64_t clock = 0;
    std::vector<uint32_t> draining;
    std::map<uint32_t, int> users;  // requests queued or running per adapter (Scheduler::uses_adapter)
    std::string err;
};

namespace {

void answer(plora_manager* m, uint64_t ticket, int status, const std::string& text) {
    auto& r = m->replies[ticket];
    r.done = true;
    r.status = status;
    r.text = text;
}

bool uses(const plora_manager* m, uint32_t id) {
    auto it = m->users.find(id);
    return it != m->users.end() && it->second > 0;
}

// src/engine.rs:604-612
void free_adapter(plora_manager* m, uint32_t id) {
    plora_free(m->h, id);
    if (m->slots) plora_slots_forget(m->slots, id);
    m->on_demand.erase(id);
    m->last_used.erase(id);
    m->users.erase(id);
}

// src/engine.rs:576-602: drops the least recently used idle on-demand adapters until at most max_cpu_loras remain
void evict(plora_manager* m) {
    const size_t cap = (size_t)m->max_cpu_loras;
    while (cap > 0 && m->on_demand.size() > cap) {
        bool found = false;
        uint32_t victim = 0;
        uint64_t oldest = 0;
        for (uint32_t id : m->on_demand) {
            if (uses(m, id)) continue;
            auto it = m->last_used.find(id);
            const uint64_t t = it == m->last_used.end() ? 0 : it->second;
            if (!found || t < oldest) {
                found = true;
                victim = id;
                oldest = t;
            }
        }
        if (!found) break;
        auto ad = m->h->adapters.find(victim);
        if (ad != m->h->adapters.end()) plora_retire(m->h, ad->second->name.c_str(), nullptr);
        free_adapter(m, victim);
    }
}

}  // namespace

extern "C" {

plora_manager_t* plora_manager_new(plora_t* h, plora_slots_t* slots, int max_cpu_loras) {
    if (!h || max_cpu_loras < 0) return nullptr;
    plora_manager* m = new plora_manager();
    m->h = h;
    m->slots = slots;
    m->max_cpu_loras = max_cpu_loras;
    return m;
}

void plora_manager_free(plora_manager_t* m) {
    if (!m) return;
    for (auto& w : m->workers)
        if (w.t.joinable()) w.t.join();
    for (auto& p : m->prepared)
        if (p.adapter) plora_adapter_drop(p.adapter);
    delete m;
}

const char* plora_manager_error(const plora_manager_t* m) { return m ? m->err.c_str() : ""; }

// Engine::start_load (src/engine.rs:505-550). The answer arrives on the ticket: at once for a name that is
// already loaded (ok when on demand, an error otherwise) or already loading (joins the wait when on demand),
// otherwise after plora_manager_finish_loads has registered what the worker thread read.
int plora_manager_load(plora_manager_t* m, const char* name, const char* path, int on_demand, uint64_t* ticket) {
    if (!m || !name || !path || !ticket) return PLORA_ERR_ARG;
    const uint64_t t = m->next_ticket++;
    *ticket = t;
    m->replies[t] = plora_manager::Reply();
    const std::string nm = name;
    uint32_t have = 0;
    if (plora_id(m->h, name, &have) == PLORA_OK) {
        if (on_demand) answer(m, t, PLORA_OK, "");
        else answer(m, t, PLORA_ERR_DUPLICATE, "adapter " + nm + " is already loaded");
        return PLORA_OK;
    }
    auto it = m->loading.find(nm);
    if (it != m->loading.end()) {
        if (on_demand) it->second.push_back(t);
        else answer(m, t, PLORA_ERR_DUPLICATE, "adapter " + nm + " is already loading");
        return PLORA_OK;
    }
    const std::string pth = path;
    const bool od = on_demand != 0;
    try {
        {
            std::lock_guard<std::mutex> g(m->mu);
            m->live_workers++;
        }
        auto done = std::make_shared<std::atomic<bool>>(false);
        std::thread th([m, nm, pth, od, done]() {
            plora_manager::Prepared p;
            p.name = nm;
            p.path = pth;
            p.on_demand = od;
            p.rc = plora_adapter_read(m->h, nm.c_str(), pth.c_str(), &p.adapter);
            if (p.rc != PLORA_OK) p.error = plora_adapter_error();
            {
                std::lock_guard<std::mutex> g(m->mu);
                m->prepared.push_back(std::move(p));
                m->live_workers--;
                m->cv.notify_all();
            }
            done->store(true);
        });
        m->workers.push_back(plora_manager::Worker{std::move(th), done});
    } catch (const std::exception& e) {
        {
            std::lock_guard<std::mutex> g(m->mu);
            m->live_workers--;
        }
        answer(m, t, PLORA_ERR_CONFIG, std::string("could not start an adapter thread: ") + e.what());
        return PLORA_OK;
    }
    m->loading[nm] = {t};
    return PLORA_OK;
}

// Engine::finish_loads (src/engine.rs:552-574): registers what the workers finished, answers the waiting
// tickets, and frees unloaded adapters no request uses any more. Returns how many adapters it registered.
int plora_manager_finish_loads(plora_manager_t* m) {
    if (!m) return -1;
    int registered = 0;
    for (;;) {
        plora_manager::Prepared p;
        {
            std::lock_guard<std::mutex> g(m->mu);
            if (m->prepared.empty()) break;
            p = std::move(m->prepared.front());
            m->prepared.pop_front();
        }
        std::vector<uint64_t> waiting;
        auto it = m->loading.find(p.name);
        if (it != m->loading.end()) {
            waiting = std::move(it->second);
            m->loading.erase(it);
        }
        int rc = p.rc;
        std::string text = p.error;
        uint32_t id = 0;
        if (rc == PLORA_OK) {
            rc = plora_insert(m->h, p.adapter, &id);  // Engine::register (src/engine.rs:490-501)
            if (rc != PLORA_OK) {
                text = plora_last_error(m->h);
                plora_adapter_drop(p.adapter);
            } else {
                registered++;
            }
        }
        if (rc == PLORA_OK && p.on_demand) {
            m->on_demand.insert(id);
            m->last_used[id] = ++m->clock;
            evict(m);
        }
        for (uint64_t t : waiting) answer(m, t, rc, text);
    }
    // threads that have handed over their result are joined and leave the list
    for (auto w = m->workers.begin(); w != m->workers.end();) {
        if (w->done->load()) {
            if (w->t.joinable()) w->t.join();
            w = m->workers.erase(w);
        } else {
            ++w;
        }
    }
    std::vector<uint32_t> still;
    for (uint32_t id : m->draining) {
        if (uses(m, id)) still.push_back(id);
        else free_adapter(m, id);
    }
    m->draining.swap(still);
    return registered;
}

// Blocks until a worker has something for finish_loads or the time runs out; 1 = something is ready.
int plora_manager_wait(plora_manager_t* m, int timeout_ms) {
    if (!m) return -1;
    std::unique_lock<std::mutex> g(m->mu);
    m->cv.wait_for(g, std::chrono::milliseconds(timeout_ms), [&] { return !m->prepared.empty() || m->live_workers == 0; });
    return m->prepared.empty() ? 0 : 1;
}

// The reply channel of a load: done = 0 while the adapter is still being read.
int plora_manager_poll(plora_manager_t* m, uint64_t ticket, int* done, int* status, char* text, int text_cap) {
    if (!m || !done || !status) return PLORA_ERR_ARG;
    auto it = m->replies.find(ticket);
    if (it == m->replies.end()) return PLORA_ERR_ARG;
    *done = it->second.done ? 1 : 0;
    *status = it->second.status;
    if (text && text_cap > 0) {
        const size_t n = std::min((size_t)text_cap - 1, it->second.text.size());
        memcpy(text, it->second.text.data(), n);
        text[n] = 0;
    }
    if (it->second.done) m->replies.erase(it);
    return PLORA_OK;
}

// Engine::loading (src/engine.rs:614-617)
int plora_manager_loading(const plora_manager_t* m) { return m && (!m->loading.empty() || !m->draining.empty()) ? 1 : 0; }

// Engine::unload_adapter (src/engine.rs:619-636): new requests can no longer name it; its memory is freed once
// the requests already using it have finished.
int plora_manager_unload(plora_manager_t* m, const char* name) {
    if (!m || !name) return PLORA_ERR_ARG;
    uint32_t id = 0;
    if (plora_retire(m->h, name, &id) != PLORA_OK || id == 0) {
        m->err = std::string("no adapter named ") + name;
        return PLORA_ERR_CONFIG;
    }
    m->on_demand.erase(id);
    if (uses(m, id)) m->draining.push_back(id);
    else free_adapter(m, id);
    return PLORA_OK;
}

// Engine::submit (src/engine.rs:638-655): a request naming an adapter that is gone is refused at once; otherwise
// the adapter counts as used (until plora_manager_release) and as recently used.
int plora_manager_submit(plora_manager_t* m, uint32_t adapter) {
    if (!m) return PLORA_ERR_ARG;
    if (adapter == 0) return PLORA_OK;
    if (!m->h->adapters.count(adapter)) {
        m->err = "the adapter was unloaded";
        return PLORA_ERR_UNKNOWN_ID;
    }
    m->last_used[adapter] = ++m->clock;
    m->users[adapter]++;
    return PLORA_OK;
}

// The request finished (Scheduler::uses_adapter turns false once none is left).
void plora_manager_release(plora_manager_t* m, uint32_t adapter) {
    if (!m || adapter == 0) return;
    auto it = m->users.find(adapter);
    if (it != m->users.end() && it->second > 0) it->second--;
}

int plora_manager_resident_on_demand(const plora_manager_t* m) { return m ? (int)m->on_demand.size() : 0; }

}  // extern "C"
