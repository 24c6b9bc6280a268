// Host model of the fused kernel's scheduling protocol, for tests that must not touch a GPU.
// TEST INFRASTRUCTURE ONLY.
//
// "Ranks" are groups of host threads with one control block each; a thread plays one CTA's
// scheduler.  The state machines are the ones of csrc/fused_prefill.cu (which follow the
// reference's src/mega_attention/kernels/sm90/fused_fa_oproj_ar.py:148-398, 1154-1177):
//
//   attention task counter -> per-row-tile head count -> ordered O_proj ready queue
//   (reserve / fill / publish in reservation order) -> ticket pop -> owner rank's ready count
//   (one arrival per rank, one byte per slot) -> claim by atomic OR of the slot's flag -> done counters -> count-out exit with
//   full-capacity clear by the last CTA -> phase/sign barrier across the ranks.
//
// Every wait is bounded as in the kernel: when the limit passes, the waiter writes a status
// {code, site, cta} once, everybody who sees a non-zero status leaves, and the launch
// returns.  The model audits exactly-once execution (a counter per attention task, O_proj
// slot and AllReduce slot) and that the control words are zero after every launch, over
// several launches with no reset in between.
//
// Faults are injected on the host only:
//   --drop-arrival R S   rank R never reports O_proj slot S to its owner (a lost message)
//   --straggler R MS     rank R starts every launch MS milliseconds late
//   --leave R L          rank R does not take part in launches >= L (a rank that left between
//                        steps); the others must time out and return, not hang
//
// Output: one JSON object on stdout.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

namespace {

using clk = std::chrono::steady_clock;
enum { C_FA_COUNTER, C_FA_DONE, C_OP_RESERVE, C_OP_PUBLISH, C_OP_CONSUME, C_OP_DONE, C_AR_DONE, C_QUIESCE, C_NUM };
enum { ST_OK = 0, ST_TIMEOUT_PUBLISH = 2, ST_TIMEOUT_NVL = 4, ST_TIMEOUT_IDLE = 6 };
enum { MODE_IDLE, MODE_FA, MODE_OPROJ, MODE_AR, MODE_DONE };

struct Config {
  int tp = 2, ctas = 6, R = 12, H = 4, nsg = 3, launches = 3, limit_ms = 300;
  int drop_rank = -1, drop_slot = -1, strag_rank = -1, strag_ms = 0, leave_rank = -1, leave_from = 0;
  // attention-task numbering, as in the kernel: 0 = one head per task; 1 = two heads that
  // share a kv head (H even, the counter steps by 2 over head ids); 2 = two heads without a
  // shared kv head (the counter numbers tasks, (H + 1) / 2 per row tile, last odd head alone)
  int pairing = 0;
};

struct Rank {
  std::atomic<uint32_t> ctrl[C_NUM];
  std::atomic<uint32_t> status{0}, status_site{0};
  std::vector<std::atomic<uint32_t>> head_ready, queue, ready_count;   // ready_count: written by peers
  std::atomic<int> nvl_signal[2];
  std::atomic<uint32_t> nvl_counter{0};
  // audit (not part of the protocol)
  std::vector<std::atomic<uint32_t>> fa_runs, op_runs, ar_runs;
  Rank(int R, int H, int total, int owned)
      : head_ready(R), queue(total), ready_count(owned), fa_runs(R * H), op_runs(total), ar_runs(owned) {
    for (auto& c : ctrl) c = 0;
    nvl_signal[0] = 0; nvl_signal[1] = 0;
  }
};

struct World {
  Config cfg;
  std::vector<Rank*> ranks;
  int total_op() const { return cfg.R * cfg.nsg; }
  int owned(int rank) const { int t = total_op() - rank; return t <= 0 ? 0 : (t + cfg.tp - 1) / cfg.tp; }
};

bool expired(clk::time_point t0, int limit_ms) {
  return std::chrono::duration_cast<std::chrono::milliseconds>(clk::now() - t0).count() > limit_ms;
}

void report(Rank& r, uint32_t code, uint32_t site) {
  uint32_t zero = 0;
  if (r.status.compare_exchange_strong(zero, code)) r.status_site = site;
}

// ---- the scheduler's three sources (same order of operations as the kernel)
bool try_fa(Rank& r, const Config& c, int num_fa, int* arg, int* nt) {
  if (c.pairing == 2) {
    const int hp = (c.H + 1) >> 1, n_tasks = (num_fa / c.H) * hp;
    if (static_cast<int>(r.ctrl[C_FA_COUNTER].load(std::memory_order_relaxed)) < n_tasks) {
      const int id = static_cast<int>(r.ctrl[C_FA_COUNTER].fetch_add(1, std::memory_order_relaxed));
      if (id < n_tasks) {
        const int head0 = 2 * (id % hp);
        *arg = (id / hp) * c.H + head0;
        *nt = std::min(2, c.H - head0);
        return true;
      }
    }
    return false;
  }
  const uint32_t step = c.pairing == 1 ? 2u : 1u;
  if (static_cast<int>(r.ctrl[C_FA_COUNTER].load(std::memory_order_relaxed)) < num_fa) {
    const uint32_t id = r.ctrl[C_FA_COUNTER].fetch_add(step, std::memory_order_relaxed);
    if (static_cast<int>(id) < num_fa) { *arg = static_cast<int>(id); *nt = static_cast<int>(step); return true; }
  }
  return false;
}

bool try_pop_oproj(Rank& r, int total_op, int* pending, int* arg) {
  if (*pending < 0) {
    const uint32_t head = r.ctrl[C_OP_CONSUME].load(std::memory_order_relaxed);
    const uint32_t tail = r.ctrl[C_OP_PUBLISH].load(std::memory_order_acquire);
    if (head >= tail) return false;
    const uint32_t t = r.ctrl[C_OP_CONSUME].fetch_add(1, std::memory_order_relaxed);
    if (static_cast<int>(t) >= total_op) return false;
    *pending = static_cast<int>(t);
    if (t >= tail && t >= r.ctrl[C_OP_PUBLISH].load(std::memory_order_acquire)) return false;
  } else if (static_cast<uint32_t>(*pending) >= r.ctrl[C_OP_PUBLISH].load(std::memory_order_acquire)) {
    return false;
  }
  *arg = static_cast<int>(r.queue[*pending].load(std::memory_order_relaxed));
  *pending = -1;
  return true;
}

// ready counts are packed one byte per slot (bit 7 = claimed), four slots per word, as in
// the kernel: arrivals add 1 << shift, the claim is an atomic OR of the flag
bool try_claim_ar(World& w, int rank, int* arg) {
  Rank& r = *w.ranks[rank];
  const int n = w.owned(rank);
  const uint32_t want = static_cast<uint32_t>(w.cfg.tp);
  for (int i = 0; i < n; ++i) {
    const int sh = (i & 3) * 8;
    if (((r.ready_count[i >> 2].load(std::memory_order_relaxed) >> sh) & 0xFFu) != want) continue;
    const uint32_t old = r.ready_count[i >> 2].fetch_or(0x80u << sh, std::memory_order_acq_rel);
    if (((old >> sh) & 0xFFu) == want) {
      *arg = i * w.cfg.tp + rank;
      return true;
    }
  }
  return false;
}

void publish_oproj(World& w, Rank& r, int row_tile) {
  const uint32_t n = static_cast<uint32_t>(w.cfg.nsg);
  const uint32_t start = r.ctrl[C_OP_RESERVE].fetch_add(n, std::memory_order_relaxed);
  for (uint32_t i = 0; i < n; ++i) r.queue[start + i].store(row_tile * n + i, std::memory_order_relaxed);
  std::atomic_thread_fence(std::memory_order_acq_rel);
  const auto t0 = clk::now();
  while (r.ctrl[C_OP_PUBLISH].load(std::memory_order_acquire) != start) {
    if (r.status.load() != 0) return;
    if (expired(t0, w.cfg.limit_ms)) { report(r, ST_TIMEOUT_PUBLISH, start); return; }
    std::this_thread::yield();
  }
  r.ctrl[C_OP_PUBLISH].fetch_add(n, std::memory_order_release);
}

void rank_barrier(World& w, int rank) {
  Rank& r = *w.ranks[rank];
  const uint32_t st = r.nvl_counter.load(std::memory_order_relaxed);
  const int phase = st & 1u, down = (st >> 1) & 1u;
  for (int peer = 0; peer < w.cfg.tp; ++peer)
    w.ranks[peer]->nvl_signal[phase].fetch_add(down ? -1 : 1, std::memory_order_release);
  r.nvl_counter.fetch_add(1, std::memory_order_relaxed);
  const int target = down ? 0 : w.cfg.tp;
  const auto t0 = clk::now();
  while (r.nvl_signal[phase].load(std::memory_order_acquire) != target) {
    if (expired(t0, w.cfg.limit_ms)) { report(r, ST_TIMEOUT_NVL, phase); break; }
    std::this_thread::yield();
  }
}

// One CTA of one rank, one launch.
void cta_main(World& w, int rank, int cta) {
  const Config& c = w.cfg;
  Rank& r = *w.ranks[rank];
  const int num_fa = c.R * c.H, total_op = w.total_op(), local_owned = w.owned(rank);
  const int role = cta % 3;                       // probe order rotates like the kernel's roles
  int pending = -1;
  bool aborted = false;
  auto idle_t0 = clk::now();
  bool idle = false;
  while (true) {
    if (r.status.load(std::memory_order_relaxed) != 0) { aborted = true; break; }
    const bool done = static_cast<int>(r.ctrl[C_FA_DONE].load(std::memory_order_acquire)) >= num_fa &&
                      static_cast<int>(r.ctrl[C_OP_DONE].load(std::memory_order_acquire)) >= total_op &&
                      static_cast<int>(r.ctrl[C_AR_DONE].load(std::memory_order_acquire)) >= local_owned;
    if (done) break;
    int mode = MODE_IDLE, arg = -1, nt = 1;
    for (int i = 0; i < 3 && mode == MODE_IDLE; ++i) {
      const int m = 1 + (role + i) % 3;
      bool ok = false;
      if (m == MODE_FA) ok = try_fa(r, c, num_fa, &arg, &nt);
      else if (m == MODE_OPROJ) ok = try_pop_oproj(r, total_op, &pending, &arg);
      else ok = try_claim_ar(w, rank, &arg);
      if (ok) mode = m;
    }
    if (mode == MODE_IDLE) {
      if (!idle) { idle = true; idle_t0 = clk::now(); }
      else if (expired(idle_t0, c.limit_ms)) { report(r, ST_TIMEOUT_IDLE, cta); aborted = true; break; }
      std::this_thread::yield();
      continue;
    }
    idle = false;
    if (mode == MODE_FA) {
      for (int i = 0; i < nt; ++i) r.fa_runs[arg + i].fetch_add(1);
      const int ft = arg / c.H;
      const uint32_t old = r.head_ready[ft].fetch_add(static_cast<uint32_t>(nt), std::memory_order_acq_rel);
      if (static_cast<int>(old) + nt == c.H) publish_oproj(w, r, ft);
      r.ctrl[C_FA_DONE].fetch_add(static_cast<uint32_t>(nt), std::memory_order_release);
    } else if (mode == MODE_OPROJ) {
      r.op_runs[arg].fetch_add(1);
      const int owner = arg % c.tp, idx = arg / c.tp;
      if (!(rank == c.drop_rank && arg == c.drop_slot))           // injected lost arrival
        w.ranks[owner]->ready_count[idx >> 2].fetch_add(1u << ((idx & 3) * 8), std::memory_order_release);
      r.ctrl[C_OP_DONE].fetch_add(1, std::memory_order_release);
    } else {
      r.ar_runs[arg / c.tp].fetch_add(1);
      r.ctrl[C_AR_DONE].fetch_add(1, std::memory_order_release);
    }
  }
  if (aborted || r.status.load() != 0) return;      // abort: no clearing, no barrier (as the kernel)
  // count-out exit: the last CTA clears the control state at full capacity and runs the
  // cross-rank barrier alone
  if (r.ctrl[C_QUIESCE].fetch_add(1, std::memory_order_acq_rel) == static_cast<uint32_t>(c.ctas - 1)) {
    for (auto& x : r.head_ready) x = 0;
    for (auto& x : r.ready_count) x = 0;
    for (int i = 0; i < C_NUM; ++i) r.ctrl[i] = 0;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    rank_barrier(w, rank);
  }
}

}  // namespace

int main(int argc, char** argv) {
  Config c;
  for (int i = 1; i < argc; ++i) {
    auto next = [&](int k) { return std::atoi(argv[i + k]); };
    if (!strcmp(argv[i], "--tp")) { c.tp = next(1); i += 1; }
    else if (!strcmp(argv[i], "--ctas")) { c.ctas = next(1); i += 1; }
    else if (!strcmp(argv[i], "--tiles")) { c.R = next(1); i += 1; }
    else if (!strcmp(argv[i], "--heads")) { c.H = next(1); i += 1; }
    else if (!strcmp(argv[i], "--nsg")) { c.nsg = next(1); i += 1; }
    else if (!strcmp(argv[i], "--pairing")) { c.pairing = next(1); i += 1; }
    else if (!strcmp(argv[i], "--launches")) { c.launches = next(1); i += 1; }
    else if (!strcmp(argv[i], "--limit-ms")) { c.limit_ms = next(1); i += 1; }
    else if (!strcmp(argv[i], "--drop-arrival")) { c.drop_rank = next(1); c.drop_slot = next(2); i += 2; }
    else if (!strcmp(argv[i], "--straggler")) { c.strag_rank = next(1); c.strag_ms = next(2); i += 2; }
    else if (!strcmp(argv[i], "--leave")) { c.leave_rank = next(1); c.leave_from = next(2); i += 2; }
    else { std::fprintf(stderr, "unknown argument %s\n", argv[i]); return 2; }
  }
  World w;
  w.cfg = c;
  const int total = c.R * c.nsg;
  for (int r = 0; r < c.tp; ++r) w.ranks.push_back(new Rank(c.R, c.H, total, w.owned(r) + 1));

  bool exactly_once = true, clean_exit = true;
  int launches_ok = 0;
  long worst_ms = 0;
  std::vector<uint32_t> first_status(c.tp, 0), first_site(c.tp, 0);
  for (int l = 0; l < c.launches; ++l) {
    const auto t0 = clk::now();
    std::vector<std::thread> th;
    for (int r = 0; r < c.tp; ++r) {
      if (r == c.leave_rank && l >= c.leave_from) continue;       // this rank is gone
      for (int k = 0; k < c.ctas; ++k)
        th.emplace_back([&w, r, k, &c]() {
          if (r == c.strag_rank) std::this_thread::sleep_for(std::chrono::milliseconds(c.strag_ms));
          cta_main(w, r, k);
        });
    }
    for (auto& t : th) t.join();
    const long ms = std::chrono::duration_cast<std::chrono::milliseconds>(clk::now() - t0).count();
    if (ms > worst_ms) worst_ms = ms;
    bool any_status = false;
    for (int r = 0; r < c.tp; ++r) {
      Rank& k = *w.ranks[r];
      if (k.status.load() != 0) {
        any_status = true;
        if (!first_status[r]) { first_status[r] = k.status.load(); first_site[r] = k.status_site.load(); }
      }
    }
    if (any_status) break;                // the host reads the status before the next launch
    ++launches_ok;
    for (int r = 0; r < c.tp; ++r) {
      Rank& k = *w.ranks[r];
      for (auto& x : k.fa_runs) { if (x.load() != 1) exactly_once = false; x = 0; }
      for (auto& x : k.op_runs) { if (x.load() != 1) exactly_once = false; x = 0; }
      for (int i = 0; i < w.owned(r); ++i) { if (k.ar_runs[i].load() != 1) exactly_once = false; k.ar_runs[i] = 0; }
      for (int i = 0; i < C_NUM; ++i) if (k.ctrl[i].load() != 0) clean_exit = false;
      for (auto& x : k.head_ready) if (x.load() != 0) clean_exit = false;
      for (auto& x : k.ready_count) if (x.load() != 0) clean_exit = false;
    }
  }
  std::printf("{\"launches_ok\": %d, \"exactly_once\": %s, \"clean_exit\": %s, \"worst_launch_ms\": %ld, "
              "\"status\": [", launches_ok, exactly_once ? "true" : "false",
              clean_exit ? "true" : "false", worst_ms);
  for (int r = 0; r < c.tp; ++r)
    std::printf("%s[%u, %u]", r ? ", " : "", first_status[r], first_site[r]);
  std::printf("]}\n");
  return 0;
}
