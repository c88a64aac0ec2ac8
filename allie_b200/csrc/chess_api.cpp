// C interface to the chess core for ctypes (allie_b200/chess/__init__.py).
#include "chess.hpp"
#include <cstdlib>

using chess::Board;
using chess::Move;

extern "C" {

void* chess_new() { return new Board(); }
void chess_free(void* h) { delete static_cast<Board*>(h); }
void* chess_copy(void* h) { return new Board(*static_cast<Board*>(h)); }
void chess_reset(void* h) { static_cast<Board*>(h)->reset(); }

// returns 1 if the move was legal and has been played
int chess_push_uci(void* h, const char* uci) {
  Board* b = static_cast<Board*>(h);
  Move m;
  if (!chess::parse_uci(uci, m)) return 0;
  std::vector<Move> legal;
  b->legal_moves(legal);
  for (const Move& l : legal)
    if (l == m) { b->push(m); return 1; }
  return 0;
}
int chess_push_id(void* h, int token_id) {
  if (token_id < 0 || token_id >= 1968) return 0;
  Board* b = static_cast<Board*>(h);
  const Move m = chess::vocab().moves[token_id];
  std::vector<Move> legal;
  b->legal_moves(legal);
  for (const Move& l : legal)
    if (l == m) { b->push(m); return 1; }
  return 0;
}
// legal moves as vocabulary token ids, in generation order; returns the count
int chess_legal_ids(void* h, int* out, int cap) {
  std::vector<Move> legal;
  static_cast<Board*>(h)->legal_moves(legal);
  int n = 0;
  for (const Move& m : legal)
    if (n < cap) out[n++] = chess::vocab().id(m);
  return int(legal.size());
}
int chess_turn(void* h) { return static_cast<Board*>(h)->turn; }
int chess_ply(void* h) { return static_cast<Board*>(h)->ply; }
int chess_is_check(void* h) { return static_cast<Board*>(h)->is_check() ? 1 : 0; }
int chess_termination(void* h) { return static_cast<Board*>(h)->termination(); }
int chess_winner(void* h) { return static_cast<Board*>(h)->winner(); }
int chess_halfmove_clock(void* h) { return static_cast<Board*>(h)->halfmove_clock; }
int chess_piece_at(void* h, int sq) {
  Board* b = static_cast<Board*>(h);
  int pt = b->piece_type_at(sq);
  if (!pt) return 0;
  return (b->occ_co[chess::WHITE] & chess::bit(sq)) ? pt : -pt;
}
// perft for the move generator tests
static unsigned long long perft_rec(Board& b, int depth) {
  std::vector<Move> legal;
  b.legal_moves(legal);
  if (depth == 1) return legal.size();
  unsigned long long n = 0;
  for (const Move& m : legal) {
    Board c = b.light_copy();
    c.apply(m);
    n += perft_rec(c, depth - 1);
  }
  return n;
}
unsigned long long chess_perft(void* h, int depth) {
  if (depth <= 0) return 1;
  Board c = static_cast<Board*>(h)->light_copy();
  return perft_rec(c, depth);
}
// vocabulary check: writes the UCI string of token `id` (5 bytes + NUL)
void chess_vocab_uci(int id, char* out) {
  std::string s = chess::move_uci(chess::vocab().moves[id]);
  std::memcpy(out, s.c_str(), s.size() + 1);
}
}

// Sets the position from a FEN string (history for repetition starts empty).  Returns 1 on success.
extern "C" int chess_set_fen(void* h, const char* fen) {
  Board* b = static_cast<Board*>(h);
  b->reset();
  for (int s = 0; s < 64; ++s) b->remove_piece(s);
  b->castling = 0;
  const char* p = fen;
  int r = 7, f = 0;
  for (; *p && *p != ' '; ++p) {
    char c = *p;
    if (c == '/') { --r; f = 0; continue; }
    if (c >= '1' && c <= '8') { f += c - '0'; continue; }
    int color = (c >= 'A' && c <= 'Z') ? chess::WHITE : chess::BLACK;
    char l = color == chess::WHITE ? char(c - 'A' + 'a') : c;
    int pt = l == 'p' ? chess::PAWN : l == 'n' ? chess::KNIGHT : l == 'b' ? chess::BISHOP
           : l == 'r' ? chess::ROOK : l == 'q' ? chess::QUEEN : l == 'k' ? chess::KING : 0;
    if (!pt || r < 0 || f > 7) return 0;
    b->set_piece(r * 8 + f, pt, color);
    ++f;
  }
  if (*p != ' ') return 0;
  ++p;
  if (*p != 'w' && *p != 'b') return 0;
  b->turn = (*p == 'w') ? chess::WHITE : chess::BLACK;
  ++p;
  if (*p == ' ') ++p;          // a FEN cut short after the side to move keeps the defaults below
  for (; *p && *p != ' '; ++p) {
    if (*p == 'K') b->castling |= chess::bit(7);
    if (*p == 'Q') b->castling |= chess::bit(0);
    if (*p == 'k') b->castling |= chess::bit(63);
    if (*p == 'q') b->castling |= chess::bit(56);
  }
  if (*p == ' ') ++p;
  b->ep_square = -1;
  if (*p && *p != '-') {
    if (p[0] < 'a' || p[0] > 'h' || p[1] < '1' || p[1] > '8') return 0;
    b->ep_square = (p[1] - '1') * 8 + (p[0] - 'a');
    p += 2;
  } else if (*p) {
    ++p;
  }
  b->halfmove_clock = 0;
  b->fullmove = 1;
  if (*p == ' ') {
    ++p;
    b->halfmove_clock = atoi(p);
    while (*p && *p != ' ') ++p;
    if (*p == ' ') b->fullmove = atoi(p + 1);
  }
  return 1;
}

// Position details a FEN string and the move-type flags need.
extern "C" {
// bit 0 = K, 1 = Q, 2 = k, 3 = q
int chess_castling_mask(void* h) {
  const Board* b = static_cast<Board*>(h);
  return ((b->castling & chess::bit(7)) ? 1 : 0) | ((b->castling & chess::bit(0)) ? 2 : 0) |
         ((b->castling & chess::bit(63)) ? 4 : 0) | ((b->castling & chess::bit(56)) ? 8 : 0);
}
int chess_ep_square(void* h) { return static_cast<Board*>(h)->ep_square; }
int chess_fullmove(void* h) { return static_cast<Board*>(h)->fullmove; }
// 1 if the current position has occurred at least `count` times since the last irreversible move
int chess_is_repetition(void* h, int count) { return static_cast<Board*>(h)->is_repetition(count) ? 1 : 0; }
}
