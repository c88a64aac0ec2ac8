// Batched AlphaZero-style MCTS over many independent game trees (one per root position).
//
// The search logic is the reference's (src/evaluation/decode.py:273-467) - PUCT with c_base/c_puct,
// values from the parent's point of view, children created eagerly for every legal move in
// generation order, first maximum wins ties, terminal leaves worth 0 (draw) or +1 (mate delivered),
// sign flip per ply on backup - but organised for a GPU evaluator: `select` walks every active tree
// to a leaf and emits one evaluation request per tree (token, position, the KV-cache slots of the
// leaf's ancestors, the leaf's legal moves); after the network ran once for the whole batch,
// `backup` expands the leaves with the returned priors and propagates the values.  Terminal leaves
// never reach the GPU: they are backed up inside `select`, which then keeps walking the same tree
// (up to the remaining simulation budget) so the evaluation batch stays full.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>

#include "chess.hpp"

namespace {

// Minimal persistent worker pool: parallel_for(n, fn) runs fn(i) for i in [0, n) on all host cores
// (the calling thread takes part).  Trees are independent, so select/backup use it per tree.
class Pool {
 public:
  Pool() {
    unsigned hc = std::thread::hardware_concurrency();
    int n = hc > 1 ? static_cast<int>(hc > 16 ? 16 : hc) - 1 : 0;
    for (int i = 0; i < n; ++i) workers_.emplace_back([this] { loop(); });
  }
  ~Pool() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& w : workers_) w.join();
  }
  void parallel_for(long n, const std::function<void(long)>& fn) {
    if (workers_.empty() || n < 8) {
      for (long i = 0; i < n; ++i) fn(i);
      return;
    }
    {
      std::lock_guard<std::mutex> lk(mu_);
      fn_ = &fn; n_ = n; next_.store(0); pending_ = static_cast<int>(workers_.size()); ++gen_;
    }
    cv_.notify_all();
    run();
    std::unique_lock<std::mutex> lk(mu_);
    done_cv_.wait(lk, [this] { return pending_ == 0; });
  }

 private:
  void run() {
    for (;;) {
      long i = next_.fetch_add(4);
      if (i >= n_) break;
      for (long j = i; j < i + 4 && j < n_; ++j) (*fn_)(j);
    }
  }
  void loop() {
    unsigned long seen = 0;
    for (;;) {
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return stop_ || gen_ != seen; });
        if (stop_) return;
        seen = gen_;
      }
      run();
      {
        std::lock_guard<std::mutex> lk(mu_);
        if (--pending_ == 0) done_cv_.notify_one();
      }
    }
  }
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable cv_, done_cv_;
  const std::function<void(long)>* fn_ = nullptr;
  long n_ = 0;
  std::atomic<long> next_{0};
  int pending_ = 0;
  unsigned long gen_ = 0;
  bool stop_ = false;
};
Pool& pool() {
  static Pool p;
  return p;
}

struct Node {
  int parent = -1;
  int move_id = -1;        // vocabulary token of the move leading here
  double prior = 0.0;      // double throughout: the oracle this is checked against computes in Python floats
  int visits = 0;
  double value_sum = 0.0;
  int first_child = -1;
  int n_children = 0;
  int depth = 0;
  int kv_slot = -1;        // KV-cache slot of this node's token (assigned when evaluated)
  double value() const { return visits ? value_sum / visits : 0.0; }
};

struct Tree {
  chess::Board root;
  std::vector<Node> nodes;
  int prefix_len = 0;       // tokens before the first searched move (ELOs, time control, game moves)
  int next_slot = 0;        // next free KV slot after the prefix
  int sims_done = 0, sims_target = 0;
  // pending evaluation
  int pending_leaf = -1;
  std::vector<int> pending_legal;
  int pending_black_to_move = 0;
  std::vector<int> path;    // scratch
};

struct Search {
  std::vector<Tree> trees;
  float c_puct = 1.25f, c_base = 19652.f;
  int depth_limit = 100;
  int max_slots = 0;
};

inline double ucb(const Search& s, const Node& parent, const Node& child, double c_puct) {
  double pb_c = std::log((parent.visits + static_cast<double>(s.c_base) + 1.0) / s.c_base) + c_puct;
  pb_c *= std::sqrt(static_cast<double>(parent.visits)) / (1.0 + child.visits);
  return pb_c * child.prior + child.value();
}

void backup(Tree& t, const std::vector<int>& path, double value) {
  for (int i = static_cast<int>(path.size()) - 1; i >= 0; --i) {
    Node& n = t.nodes[path[i]];
    n.value_sum += value;
    n.visits += 1;
    value = -value;
  }
}

void expand(Tree& t, int node, const int* legal, const float* priors, int n) {
  const int first = static_cast<int>(t.nodes.size());
  const int depth = t.nodes[node].depth + 1;
  t.nodes.resize(first + n);
  for (int i = 0; i < n; ++i) {
    Node& c = t.nodes[first + i];
    c = Node();
    c.parent = node;
    c.move_id = legal[i];
    c.prior = priors[i];
    c.depth = depth;
  }
  t.nodes[node].first_child = first;
  t.nodes[node].n_children = n;
}

// board at `node`: the root position plus the moves on the path
chess::Board board_at(const Tree& t, const std::vector<int>& path) {
  chess::Board b = t.root;   // keeps the repetition history of the real game
  for (size_t i = 1; i < path.size(); ++i) b.push(chess::vocab().moves[t.nodes[path[i]].move_id]);
  return b;
}

}  // namespace

extern "C" {

void* mcts_create(int n_trees, float c_puct, float c_base, int depth_limit, int max_slots) {
  Search* s = new Search();
  s->trees.resize(n_trees);
  s->c_puct = c_puct; s->c_base = c_base; s->depth_limit = depth_limit; s->max_slots = max_slots;
  return s;
}
void mcts_destroy(void* h) { delete static_cast<Search*>(h); }

// Root = start position + `n_moves` vocabulary tokens.  prefix_len = tokens of the whole prompt.
// Returns the number of legal moves at the root (written to out_legal), 0 if the root is terminal,
// -1 on an illegal move in the prefix.
int mcts_set_root(void* h, int t, const int* move_ids, int n_moves, int prefix_len, int sims_target,
                  int* out_legal, int cap) {
  Search* s = static_cast<Search*>(h);
  Tree& tr = s->trees[t];
  tr.root.reset();
  std::vector<chess::Move> legal;
  for (int i = 0; i < n_moves; ++i) {
    if (move_ids[i] < 0 || move_ids[i] >= 1968) return -1;
    const chess::Move m = chess::vocab().moves[move_ids[i]];
    tr.root.legal_moves(legal);
    if (std::find(legal.begin(), legal.end(), m) == legal.end()) return -1;
    tr.root.push(m);
  }
  tr.nodes.clear();
  tr.nodes.emplace_back();
  tr.prefix_len = prefix_len;
  tr.next_slot = prefix_len;
  tr.sims_done = 0;
  tr.sims_target = sims_target;
  tr.pending_leaf = -1;
  if (tr.root.is_game_over()) return 0;
  tr.root.legal_moves(legal);
  int n = 0;
  for (const auto& m : legal)
    if (n < cap) out_legal[n++] = chess::vocab().id(m);
  return static_cast<int>(legal.size());
}

int mcts_root_turn(void* h, int t) { return static_cast<Search*>(h)->trees[t].root.turn; }

// Children of the root from the prefill evaluation (no backup, like the reference's first
// evaluate_node(root) call).
void mcts_expand_root(void* h, int t, const int* legal, const float* priors, int n) {
  Tree& tr = static_cast<Search*>(h)->trees[t];
  expand(tr, 0, legal, priors, n);
}

void mcts_set_budget(void* h, int t, int sims_target) { static_cast<Search*>(h)->trees[t].sims_target = sims_target; }
int mcts_sims_done(void* h, int t) { return static_cast<Search*>(h)->trees[t].sims_done; }

// One selection round.  For every tree with budget left, walk to a leaf; terminal leaves are backed
// up on the spot and the walk repeats.  Per tree t the outputs are:
//   need_eval[t]           1 if a network evaluation is requested
//   tok[t], pos[t]         token id and position id of the leaf's move
//   slot[t]                KV-cache slot to store the leaf's keys/values in
//   anc[t*anc_stride + i]  KV slots of the ancestors below the root, oldest first, then the leaf's
//   n_anc[t]               how many of those (= leaf depth)
//   legal[t*legal_stride + i], n_legal[t]   the leaf's legal moves (vocabulary ids, generation order)
// c_puct_per_tree may be null (use the global constant).  Returns the number of requests.
int mcts_select(void* h, const float* c_puct_per_tree, int* need_eval, int* tok, int* pos, int* slot,
                int* anc, int anc_stride, int* n_anc, int* legal, int legal_stride, int* n_legal) {
  Search* s = static_cast<Search*>(h);
  std::atomic<int> requests{0};
  // trees are independent: walk them on all host cores
  pool().parallel_for(static_cast<long>(s->trees.size()), [&](long ti) {
    std::vector<chess::Move> moves;
    Tree& t = s->trees[ti];
    need_eval[ti] = 0;
    n_anc[ti] = 0;
    n_legal[ti] = 0;
    t.pending_leaf = -1;
    const double cp = c_puct_per_tree ? c_puct_per_tree[ti] : s->c_puct;
    while (t.sims_done < t.sims_target && !t.nodes.empty() && t.nodes[0].n_children > 0) {
      std::vector<int>& path = t.path;
      path.clear();
      int node = 0;
      path.push_back(0);
      while (t.nodes[node].n_children > 0 && static_cast<int>(path.size()) <= s->depth_limit) {
        const Node& p = t.nodes[node];
        int best = p.first_child;
        double best_score = ucb(*s, p, t.nodes[best], cp);
        for (int c = p.first_child + 1; c < p.first_child + p.n_children; ++c) {
          const double sc = ucb(*s, p, t.nodes[c], cp);
          if (sc > best_score) { best_score = sc; best = c; }
        }
        node = best;
        path.push_back(node);
      }
      chess::Board b = board_at(t, path);
      const int term = b.termination();
      if (term != 0) {
        backup(t, path, term == 1 ? 1.0 : 0.0);
        ++t.sims_done;
        continue;
      }
      if (t.nodes[node].n_children > 0 || t.next_slot >= s->max_slots ||
          static_cast<int>(path.size()) - 1 > anc_stride) {
        // depth limit reached on an expanded node (or the cache is full): the reference would
        // re-evaluate the position; its value is already known here, so reuse the stored mean
        backup(t, path, t.nodes[node].visits ? t.nodes[node].value() : 0.0);
        ++t.sims_done;
        continue;
      }
      // request an evaluation of this leaf
      Node& leaf = t.nodes[node];
      leaf.kv_slot = t.next_slot++;
      need_eval[ti] = 1;
      tok[ti] = leaf.move_id;
      pos[ti] = t.prefix_len + leaf.depth - 1;
      slot[ti] = leaf.kv_slot;
      int na = 0;
      for (size_t i = 1; i < path.size(); ++i) anc[ti * anc_stride + na++] = t.nodes[path[i]].kv_slot;
      n_anc[ti] = na;
      b.legal_moves(moves);
      t.pending_legal.clear();
      int nl = 0;
      for (const auto& m : moves) {
        const int id = chess::vocab().id(m);
        t.pending_legal.push_back(id);
        if (nl < legal_stride) legal[ti * legal_stride + nl++] = id;
      }
      n_legal[ti] = static_cast<int>(moves.size());
      t.pending_leaf = node;
      t.pending_black_to_move = b.turn == chess::BLACK;
      requests.fetch_add(1);
      break;
    }
  });
  return requests.load();
}

// Consumes the evaluation of every tree that requested one: priors[t*stride + i] over the leaf's
// legal moves (already soft-maxed), value[t] = raw value-head output (white advantage).
void mcts_backup(void* h, const float* priors, int stride, const float* value, int dummy_value) {
  Search* s = static_cast<Search*>(h);
  pool().parallel_for(static_cast<long>(s->trees.size()), [&](long ti) {
    Tree& t = s->trees[ti];
    if (t.pending_leaf < 0) return;
    const int leaf = t.pending_leaf;
    expand(t, leaf, t.pending_legal.data(), priors + ti * stride, static_cast<int>(t.pending_legal.size()));
    // value from the parent's point of view: + if black is to move at the leaf
    const double v = dummy_value ? 0.0 : (t.pending_black_to_move ? double(value[ti]) : -double(value[ti]));
    std::vector<int>& path = t.path;
    path.clear();
    for (int n = leaf; n >= 0; n = t.nodes[n].parent) path.push_back(n);
    std::reverse(path.begin(), path.end());
    backup(t, path, v);
    ++t.sims_done;
    t.pending_leaf = -1;
  });
}

// Root statistics in root-child order.  Returns the number of children.
int mcts_root_stats(void* h, int t, int* move_ids, int* visits, float* priors, float* values, int cap) {
  Tree& tr = static_cast<Search*>(h)->trees[t];
  if (tr.nodes.empty()) return 0;
  const Node& r = tr.nodes[0];
  int n = 0;
  for (int c = r.first_child; c < r.first_child + r.n_children && n < cap; ++c, ++n) {
    move_ids[n] = tr.nodes[c].move_id;
    visits[n] = tr.nodes[c].visits;
    priors[n] = static_cast<float>(tr.nodes[c].prior);
    values[n] = static_cast<float>(tr.nodes[c].value());
  }
  return r.n_children;
}

int mcts_node_count(void* h, int t) { return static_cast<int>(static_cast<Search*>(h)->trees[t].nodes.size()); }
}
