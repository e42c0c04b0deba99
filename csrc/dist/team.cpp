// Rank control plane: one owner, N rank worker threads, lock-step command broadcast with
// deadlines, sticky fail-closed failure, plus an in-process fake collective backend used to
// test the protocol (and failure handling) on CPU ranks.
//
// * Every command goes to ALL ranks; the owner waits for ALL replies before the next command,
//   so per-rank collective sequences can never diverge.
// * Every command has a deadline (fast or heavy).  The first error, timeout or lost rank is
//   recorded (rank, code) and is sticky: later broadcasts fail fast without touching the ranks.
// * Failure injection for tests happens here, on the host: drop a reply, delay it, make the
//   handler's result an error, or retire the rank thread.
// Behavioural contract: crates/orinfer-engine/src/models/deepseek_v41/team/channel.rs:12-33,
// 68-169 (deadlines, fail-closed transport) and team.rs:971-1060 of the reference; the fake
// backend plays the role of its fake ACL runtime (tests/fixtures/ascend_runtime.c).
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

namespace {

using Clock = std::chrono::steady_clock;
using Handler = long long (*)(void* user, int rank, int opcode, const long long* args, int nargs,
                              int* status);

enum Result { OK = 0, TIMEOUT = -1, RANK_ERROR = -2, DISCONNECTED = -3, STICKY = -4 };
enum Inject { NONE = 0, DROP_REPLY = 1, DELAY_MS = 2, ERROR_CODE = 3, EXIT_THREAD = 4 };

struct Command {
  long long serial;
  int opcode;
  std::vector<long long> args;
  bool quit = false;
};

struct Reply {
  long long serial;
  long long value;
  int status;
};

struct Rank {
  std::mutex m;
  std::condition_variable cv;
  std::deque<Command> inbox;
  std::deque<Reply> outbox;
  std::thread thread;
  std::atomic<bool> alive{true};
  // injection: applies to the command with ordinal `at` (0 = next), then clears
  int inject_kind = NONE;
  long long inject_value = 0;
  long long inject_at = 0;
  long long handled = 0;
};

struct Team {
  int n;
  Handler handler;
  void* user;
  int fast_ms, heavy_ms;
  std::vector<Rank*> ranks;
  std::mutex owner;
  std::condition_variable reply_cv;
  std::mutex reply_m;
  long long serial = 0;
  int failed_rank = -1;
  int failed_code = 0;
  std::atomic<bool> failed{false};
};

void fail(Team* t, int rank, int code) {
  bool expected = false;
  if (t->failed.compare_exchange_strong(expected, true)) {
    t->failed_rank = rank;
    t->failed_code = code;
  }
}

void worker(Team* t, int r) {
  Rank* rk = t->ranks[r];
  for (;;) {
    Command c;
    {
      std::unique_lock<std::mutex> lk(rk->m);
      rk->cv.wait(lk, [&] { return !rk->inbox.empty(); });
      c = std::move(rk->inbox.front());
      rk->inbox.pop_front();
    }
    if (c.quit) break;
    int kind = NONE;
    long long val = 0;
    {
      std::lock_guard<std::mutex> lk(rk->m);
      if (rk->inject_kind != NONE && rk->handled >= rk->inject_at) {
        kind = rk->inject_kind;
        val = rk->inject_value;
        rk->inject_kind = NONE;
      }
      ++rk->handled;
    }
    if (kind == EXIT_THREAD) break;                    // the rank disappears without a reply
    int status = 0;
    long long value = t->handler(t->user, r, c.opcode, c.args.data(),
                                 static_cast<int>(c.args.size()), &status);
    if (kind == DELAY_MS) std::this_thread::sleep_for(std::chrono::milliseconds(val));
    if (kind == ERROR_CODE) status = static_cast<int>(val);
    if (kind == DROP_REPLY) continue;
    {
      std::lock_guard<std::mutex> lk(t->reply_m);
      rk->outbox.push_back(Reply{c.serial, value, status});
    }
    t->reply_cv.notify_all();
  }
  rk->alive = false;
  t->reply_cv.notify_all();
}

// ---- fake collective backend: N threads meet at a generation barrier with a deadline
struct FakeComm {
  int n;
  std::mutex m;
  std::condition_variable cv;
  long long generation = 0;
  int arrived = 0;
  std::vector<const double*> src;
  std::vector<double> sum;
  std::vector<int> fail_code;       // per rank: non-zero => that rank's next call fails
  bool broken = false;
  long long calls = 0;
};

}  // namespace

extern "C" {

void* orinfer_team_create(int ranks, Handler handler, void* user, int fast_ms, int heavy_ms) {
  if (ranks < 1 || ranks > 64 || handler == nullptr) return nullptr;
  Team* t = new Team();
  t->n = ranks;
  t->handler = handler;
  t->user = user;
  t->fast_ms = fast_ms;
  t->heavy_ms = heavy_ms;
  for (int r = 0; r < ranks; ++r) t->ranks.push_back(new Rank());
  for (int r = 0; r < ranks; ++r) t->ranks[r]->thread = std::thread(worker, t, r);
  return t;
}

// Sends (opcode, args) to every rank and waits for every reply.  replies[r] receives rank r's
// value.  Returns 0, or TIMEOUT / RANK_ERROR / DISCONNECTED for the first failure (which
// becomes sticky), or STICKY when the team had already failed.
int orinfer_team_broadcast(void* h, int opcode, const long long* args, int nargs, int heavy,
                           long long* replies) {
  Team* t = static_cast<Team*>(h);
  std::lock_guard<std::mutex> own(t->owner);
  if (t->failed) return STICKY;
  const long long serial = ++t->serial;
  for (int r = 0; r < t->n; ++r) {
    Rank* rk = t->ranks[r];
    if (!rk->alive) {
      fail(t, r, DISCONNECTED);
      return DISCONNECTED;
    }
    Command c;
    c.serial = serial;
    c.opcode = opcode;
    c.args.assign(args, args + nargs);
    {
      std::lock_guard<std::mutex> lk(rk->m);
      rk->inbox.push_back(std::move(c));
    }
    rk->cv.notify_one();
  }
  const auto deadline = Clock::now() + std::chrono::milliseconds(heavy ? t->heavy_ms : t->fast_ms);
  std::vector<bool> got(t->n, false);
  int missing = t->n;
  std::unique_lock<std::mutex> lk(t->reply_m);
  while (missing > 0) {
    for (int r = 0; r < t->n; ++r) {
      Rank* rk = t->ranks[r];
      while (!rk->outbox.empty()) {
        Reply rep = rk->outbox.front();
        rk->outbox.pop_front();
        if (rep.serial != serial) continue;            // a late reply of an abandoned command
        if (rep.status != 0) {
          fail(t, r, rep.status);
          return RANK_ERROR;
        }
        if (!got[r]) {
          got[r] = true;
          --missing;
          if (replies) replies[r] = rep.value;
        }
      }
      if (!got[r] && !rk->alive) {
        fail(t, r, DISCONNECTED);
        return DISCONNECTED;
      }
    }
    if (missing == 0) break;
    if (t->reply_cv.wait_until(lk, deadline) == std::cv_status::timeout) {
      for (int r = 0; r < t->n; ++r)
        if (!got[r]) {
          fail(t, r, TIMEOUT);
          break;
        }
      return TIMEOUT;
    }
  }
  return OK;
}

// 0 when healthy; else 1 and (*rank, *code) of the first failure.
int orinfer_team_failure(void* h, int* rank, int* code) {
  Team* t = static_cast<Team*>(h);
  if (!t->failed) return 0;
  if (rank) *rank = t->failed_rank;
  if (code) *code = t->failed_code;
  return 1;
}

// Arms one injection on `rank`: it hits the rank's command number `at` (counted from the
// rank's start) or the next one if that number has passed.
void orinfer_team_inject(void* h, int rank, int kind, long long value, long long at) {
  Team* t = static_cast<Team*>(h);
  Rank* rk = t->ranks[rank];
  std::lock_guard<std::mutex> lk(rk->m);
  rk->inject_kind = kind;
  rk->inject_value = value;
  rk->inject_at = at;
}

void orinfer_team_destroy(void* h) {
  Team* t = static_cast<Team*>(h);
  for (Rank* rk : t->ranks) {
    Command c;
    c.quit = true;
    {
      std::lock_guard<std::mutex> lk(rk->m);
      rk->inbox.push_back(std::move(c));
    }
    rk->cv.notify_one();
  }
  for (Rank* rk : t->ranks) {
    if (rk->thread.joinable()) rk->thread.join();
    delete rk;
  }
  delete t;
}

// ---- fake collectives (sum all-reduce of doubles among `ranks` threads)
void* orinfer_fakecomm_create(int ranks) {
  FakeComm* c = new FakeComm();
  c->n = ranks;
  c->src.assign(ranks, nullptr);
  c->fail_code.assign(ranks, 0);
  return c;
}
void orinfer_fakecomm_destroy(void* h) { delete static_cast<FakeComm*>(h); }

// The next call of `rank` returns `code` without joining (the peers then time out).
void orinfer_fakecomm_fail_next(void* h, int rank, int code) {
  FakeComm* c = static_cast<FakeComm*>(h);
  std::lock_guard<std::mutex> lk(c->m);
  c->fail_code[rank] = code;
}

long long orinfer_fakecomm_calls(void* h) { return static_cast<FakeComm*>(h)->calls; }

// In-place sum over ranks.  0 on success, the injected code for a failing rank, -1 when the
// other ranks did not arrive within timeout_ms, -5 when the communicator is already broken.
int orinfer_fakecomm_all_reduce(void* h, int rank, double* buf, int count, int timeout_ms) {
  FakeComm* c = static_cast<FakeComm*>(h);
  std::unique_lock<std::mutex> lk(c->m);
  if (c->broken) return -5;
  if (c->fail_code[rank]) {
    const int code = c->fail_code[rank];
    c->fail_code[rank] = 0;
    return code;
  }
  const long long gen = c->generation;
  c->src[rank] = buf;
  if (++c->arrived == c->n) {
    c->sum.assign(count, 0.0);
    for (int r = 0; r < c->n; ++r)
      for (int i = 0; i < count; ++i) c->sum[i] += c->src[r][i];
    c->arrived = 0;
    ++c->generation;
    ++c->calls;
    c->cv.notify_all();
  } else {
    const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
    if (!c->cv.wait_until(lk, deadline, [&] { return c->generation != gen || c->broken; })) {
      c->broken = true;                               // a peer never joined: poison the group
      c->cv.notify_all();
      return -1;
    }
    if (c->broken) return -5;
  }
  std::memcpy(buf, c->sum.data(), sizeof(double) * count);
  return 0;
}

}  // extern "C"
