// PGN movetext -> UCI moves and per-move seconds, for the data preparation step
// (allie_b200/etl/pgn.py).  One call per game: tokenises the movetext, reads the clock comments
// ([%clk h:mm:ss]), resolves every SAN token against the legal moves of the running position
// and plays it.  The reference does this in Python through python-chess's PGN reader
// (src/data/process-lichess.py:30-47); a month of Lichess games is tens of millions of calls.
#include "chess.hpp"
#include <cctype>
#include <cstdlib>

namespace {

using chess::Board;
using chess::Move;

// Resolves one SAN token (check marks and annotations allowed).  True when exactly one legal move fits.
bool resolve_san(const Board& b, const char* tok, size_t n, Move& out) {
  while (n && (tok[n - 1] == '+' || tok[n - 1] == '#' || tok[n - 1] == '!' || tok[n - 1] == '?')) --n;
  if (!n || n > 15) return false;
  std::vector<Move> legal;
  b.legal_moves(legal);
  std::string s(tok, n);
  if (s == "O-O" || s == "0-0" || s == "O-O-O" || s == "0-0-0") {
    const bool king_side = s.size() == 3;
    const int from = b.turn == chess::WHITE ? 4 : 60;
    Move want;
    want.from = uint8_t(from);
    want.to = uint8_t(king_side ? from + 2 : from - 2);
    for (const Move& m : legal)
      if (m == want && b.piece_type_at(m.from) == chess::KING) { out = m; return true; }
    return false;
  }
  int promo = 0;
  size_t eq = s.find('=');
  if (eq != std::string::npos) {
    if (eq + 1 >= s.size()) return false;
    switch (std::tolower(s[eq + 1])) {
      case 'n': promo = chess::KNIGHT; break;
      case 'b': promo = chess::BISHOP; break;
      case 'r': promo = chess::ROOK; break;
      case 'q': promo = chess::QUEEN; break;
      default: return false;
    }
    s.resize(eq);
  }
  if (s.empty()) return false;
  int piece = chess::PAWN;
  switch (s[0]) {
    case 'N': piece = chess::KNIGHT; break;
    case 'B': piece = chess::BISHOP; break;
    case 'R': piece = chess::ROOK; break;
    case 'Q': piece = chess::QUEEN; break;
    case 'K': piece = chess::KING; break;
    default: break;
  }
  std::string body = piece == chess::PAWN ? s : s.substr(1);
  std::string clean;
  for (char c : body)
    if (c != 'x') clean += c;
  if (clean.size() < 2) return false;
  const char df = clean[clean.size() - 2], dr = clean[clean.size() - 1];
  if (df < 'a' || df > 'h' || dr < '1' || dr > '8') return false;
  const int dest = (dr - '1') * 8 + (df - 'a');
  const std::string dis = clean.substr(0, clean.size() - 2);
  int hits = 0;
  for (const Move& m : legal) {
    if (m.to != dest || m.promo != promo || b.piece_type_at(m.from) != piece) continue;
    const char ff = char('a' + chess::file_of(m.from)), fr = char('1' + chess::rank_of(m.from));
    bool ok = true;
    for (char c : dis)
      if (c != ff && c != fr) ok = false;
    if (!ok) continue;
    out = m;
    ++hits;
  }
  return hits == 1;
}

}  // namespace

extern "C" {

// Writes the SAN text of a legal move given as UCI text (minimal disambiguation, "+" / "#" suffix),
// at most 8 characters + NUL.  Returns 1 on success, 0 when the move is not legal here.
int chess_san(void* h, const char* uci, char* san_out) {
  const Board& b = *static_cast<Board*>(h);
  Move m;
  if (!chess::parse_uci(uci, m)) return 0;
  std::vector<Move> legal;
  b.legal_moves(legal);
  bool found = false;
  for (const Move& l : legal) found = found || l == m;
  if (!found) return 0;
  const int pt = b.piece_type_at(m.from);
  std::string s;
  if (pt == chess::KING && std::abs(chess::file_of(m.to) - chess::file_of(m.from)) == 2) {
    s = chess::file_of(m.to) > chess::file_of(m.from) ? "O-O" : "O-O-O";
  } else {
    const bool capture = (b.occ & chess::bit(m.to)) || b.is_en_passant(m);
    const char ff = char('a' + chess::file_of(m.from)), fr = char('1' + chess::rank_of(m.from));
    if (pt == chess::PAWN) {
      if (capture) { s += ff; s += 'x'; }
    } else {
      s += " PNBRQK"[pt];
      bool others = false, file_clash = false, rank_clash = false;
      for (const Move& l : legal) {
        if (l.to != m.to || l.from == m.from || b.piece_type_at(l.from) != pt) continue;
        others = true;
        if (chess::file_of(l.from) == chess::file_of(m.from)) file_clash = true;
        if (chess::rank_of(l.from) == chess::rank_of(m.from)) rank_clash = true;
      }
      if (others) {
        if (!file_clash) s += ff;
        else if (!rank_clash) s += fr;
        else { s += ff; s += fr; }
      }
      if (capture) s += 'x';
    }
    s += char('a' + chess::file_of(m.to));
    s += char('1' + chess::rank_of(m.to));
    if (m.promo) { s += '='; s += " PNBRQK"[m.promo]; }
  }
  Board next = b.light_copy();
  next.apply(m);
  if (next.is_check()) s += next.has_legal_move() ? '+' : '#';
  std::memcpy(san_out, s.c_str(), s.size() + 1);
  return 1;
}

// Resolves one SAN move without playing it; writes its UCI text.  Returns 1 on success.
int chess_parse_san(void* h, const char* san, char* uci_out) {
  Move m;
  if (!resolve_san(*static_cast<Board*>(h), san, std::strlen(san), m)) return 0;
  std::string u = chess::move_uci(m);
  std::memcpy(uci_out, u.c_str(), u.size() + 1);
  return 1;
}

// Plays one SAN move on the board; writes its UCI text (at most 5 characters + NUL).  Returns 1 on
// success, 0 when the token fits no legal move or more than one.
int chess_push_san(void* h, const char* san, char* uci_out) {
  Board* b = static_cast<Board*>(h);
  Move m;
  if (!resolve_san(*b, san, std::strlen(san), m)) return 0;
  std::string u = chess::move_uci(m);
  std::memcpy(uci_out, u.c_str(), u.size() + 1);
  b->push(m);
  return 1;
}

// Parses the movetext of one game that starts from the initial position.
//   base, inc      time control in seconds (the clock of both sides starts at `base`)
//   uci_out        receives the moves as space separated UCI text (NUL terminated), capacity `cap`
//   seconds_out    receives the seconds spent on each move that carries a clock comment:
//                  max(0, previous clock of that side - new clock + inc)
// Returns the number of moves, or -1 for an unresolvable move / a full buffer; *n_seconds is the
// number of entries written to seconds_out (callers drop games where it differs from the move count).
int pgn_parse_movetext(const char* text, int base, int inc, char* uci_out, int cap, int* seconds_out,
                       int max_moves, int* n_seconds) {
  Board board;
  int n_moves = 0, n_secs = 0, used = 0;
  long long clocks[2] = {base, base};
  const char* p = text;
  *n_seconds = 0;
  if (cap > 0) uci_out[0] = 0;
  while (*p) {
    while (*p && std::isspace(static_cast<unsigned char>(*p))) ++p;
    if (!*p) break;
    if (*p == '{') {
      const char* end = std::strchr(p, '}');
      if (!end) end = p + std::strlen(p);
      const char* c = std::strstr(p, "[%clk ");
      if (c && c < end && n_moves > 0) {
        int hh = 0, mm = 0, ss = 0;
        if (std::sscanf(c + 6, "%d:%d:%d", &hh, &mm, &ss) == 3 && n_secs < max_moves) {
          const int side = (n_moves - 1) % 2;
          const long long now = hh * 3600LL + mm * 60LL + ss;
          const long long spent = clocks[side] - now + inc;
          seconds_out[n_secs++] = int(spent > 0 ? spent : 0);
          clocks[side] = now;
        }
      }
      p = *end ? end + 1 : end;
      continue;
    }
    const char* start = p;
    while (*p && !std::isspace(static_cast<unsigned char>(*p))) ++p;
    size_t n = size_t(p - start);
    std::string tok(start, n);
    if (tok == "1-0" || tok == "0-1" || tok == "1/2-1/2" || tok == "*") continue;
    if (std::isdigit(static_cast<unsigned char>(tok[0]))) {
      // a move number ("12." / "12...") possibly glued to the move ("12.e4")
      size_t i = 0;
      while (i < tok.size() && std::isdigit(static_cast<unsigned char>(tok[i]))) ++i;
      size_t j = i;
      while (j < tok.size() && tok[j] == '.') ++j;
      if (j > i) tok = tok.substr(j);
      if (tok.empty()) continue;
    }
    Move m;
    if (!resolve_san(board, tok.c_str(), tok.size(), m)) return -1;
    std::string u = chess::move_uci(m);
    if (n_moves >= max_moves || used + int(u.size()) + 2 > cap) return -1;
    if (n_moves) uci_out[used++] = ' ';
    std::memcpy(uci_out + used, u.c_str(), u.size());
    used += int(u.size());
    uci_out[used] = 0;
    board.push(m);
    ++n_moves;
  }
  *n_seconds = n_secs;
  return n_moves;
}
}
