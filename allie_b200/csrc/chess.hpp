// Bitboard chess: legal move generation, make-move, terminal detection.
//
// Two properties matter beyond correctness:
//  * moves come out in the same order as python-chess's `Board.legal_moves`, because the search
//    breaks PUCT ties by "first legal move wins" (reference src/evaluation/decode.py:381-384 relies
//    on python-chess order): non-pawn piece moves scanning squares from h8 down to a1, castling,
//    pawn captures, single pushes, double pushes, en passant; when in check: king evasions first,
//    then blocks/captures of a single checker;
//  * `is_game_over` has python-chess semantics without draw claims: checkmate, stalemate,
//    insufficient material, the 75-move rule and fivefold repetition.
// Header-only so the batched MCTS can inline it.
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace chess {

using BB = uint64_t;
enum Color : int { BLACK = 0, WHITE = 1 };
enum PieceType : int { NONE = 0, PAWN = 1, KNIGHT = 2, BISHOP = 3, ROOK = 4, QUEEN = 5, KING = 6 };

inline BB bit(int sq) { return BB(1) << sq; }
inline int msb(BB b) { return 63 - __builtin_clzll(b); }
inline int lsb(BB b) { return __builtin_ctzll(b); }
inline int popcount(BB b) { return __builtin_popcountll(b); }
inline int file_of(int sq) { return sq & 7; }
inline int rank_of(int sq) { return sq >> 3; }

constexpr BB BB_RANK_1 = 0xFFull, BB_RANK_2 = 0xFF00ull, BB_RANK_3 = 0xFF0000ull,
             BB_RANK_4 = 0xFF000000ull, BB_RANK_5 = 0xFF00000000ull, BB_RANK_6 = 0xFF0000000000ull,
             BB_RANK_7 = 0xFF000000000000ull, BB_RANK_8 = 0xFF00000000000000ull;
constexpr BB BB_LIGHT = 0x55AA55AA55AA55AAull, BB_DARK = 0xAA55AA55AA55AA55ull;
constexpr BB BB_FILE_A = 0x0101010101010101ull, BB_FILE_H = 0x8080808080808080ull;

struct Move {
  uint8_t from = 0, to = 0, promo = 0;  // promo: PieceType or 0
  bool operator==(const Move& o) const { return from == o.from && to == o.to && promo == o.promo; }
};

struct Tables {
  BB knight[64], king[64], pawn_att[2][64];
  BB ray[64][64];      // full line through both squares (0 if not aligned)
  BB between[64][64];  // squares strictly between
  Tables() {
    for (int s = 0; s < 64; ++s) {
      int f = file_of(s), r = rank_of(s);
      knight[s] = king[s] = pawn_att[0][s] = pawn_att[1][s] = 0;
      const int kd[8][2] = {{1, 2}, {2, 1}, {-1, 2}, {-2, 1}, {1, -2}, {2, -1}, {-1, -2}, {-2, -1}};
      for (auto& d : kd) {
        int nf = f + d[0], nr = r + d[1];
        if (nf >= 0 && nf < 8 && nr >= 0 && nr < 8) knight[s] |= bit(nr * 8 + nf);
      }
      for (int df = -1; df <= 1; ++df)
        for (int dr = -1; dr <= 1; ++dr) {
          if (!df && !dr) continue;
          int nf = f + df, nr = r + dr;
          if (nf >= 0 && nf < 8 && nr >= 0 && nr < 8) king[s] |= bit(nr * 8 + nf);
        }
      for (int df = -1; df <= 1; df += 2) {
        int nf = f + df;
        if (nf < 0 || nf > 7) continue;
        if (r + 1 < 8) pawn_att[WHITE][s] |= bit((r + 1) * 8 + nf);
        if (r - 1 >= 0) pawn_att[BLACK][s] |= bit((r - 1) * 8 + nf);
      }
    }
    for (int a = 0; a < 64; ++a)
      for (int b = 0; b < 64; ++b) {
        ray[a][b] = between[a][b] = 0;
        if (a == b) continue;
        int df = file_of(b) - file_of(a), dr = rank_of(b) - rank_of(a);
        if (!(df == 0 || dr == 0 || df == dr || df == -dr)) continue;
        int sf = (df > 0) - (df < 0), sr = (dr > 0) - (dr < 0);
        BB line = bit(a);
        for (int f = file_of(a) + sf, r = rank_of(a) + sr; f >= 0 && f < 8 && r >= 0 && r < 8; f += sf, r += sr)
          line |= bit(r * 8 + f);
        for (int f = file_of(a) - sf, r = rank_of(a) - sr; f >= 0 && f < 8 && r >= 0 && r < 8; f -= sf, r -= sr)
          line |= bit(r * 8 + f);
        ray[a][b] = line;
        BB bt = 0;
        for (int f = file_of(a) + sf, r = rank_of(a) + sr; r * 8 + f != b; f += sf, r += sr) bt |= bit(r * 8 + f);
        between[a][b] = bt;
      }
  }
};
inline const Tables& T() {
  static const Tables t;
  return t;
}

inline BB slide(int sq, BB occ, const int (*dirs)[2], int nd) {
  BB att = 0;
  for (int i = 0; i < nd; ++i) {
    int f = file_of(sq) + dirs[i][0], r = rank_of(sq) + dirs[i][1];
    while (f >= 0 && f < 8 && r >= 0 && r < 8) {
      BB b = bit(r * 8 + f);
      att |= b;
      if (occ & b) break;
      f += dirs[i][0];
      r += dirs[i][1];
    }
  }
  return att;
}
inline BB rook_att(int sq, BB occ) {
  static const int d[4][2] = {{1, 0}, {-1, 0}, {0, 1}, {0, -1}};
  return slide(sq, occ, d, 4);
}
inline BB bishop_att(int sq, BB occ) {
  static const int d[4][2] = {{1, 1}, {-1, 1}, {1, -1}, {-1, -1}};
  return slide(sq, occ, d, 4);
}

// What repetition detection compares (python-chess `_transposition_key`).
struct PosKey {
  BB pawns, knights, bishops, rooks, queens, kings, white, black, castling;
  int turn, ep;
  bool operator==(const PosKey& o) const { return std::memcmp(this, &o, sizeof(PosKey)) == 0; }
};

struct Board {
  BB pawns, knights, bishops, rooks, queens, kings;
  BB occ_co[2], occ;
  BB castling;       // rook squares that still carry castling rights
  int turn;          // WHITE / BLACK
  int ep_square;     // -1 if none (set after every double push, like python-chess)
  int halfmove_clock, fullmove;
  int ply = 0;
  // per-ply history since the game start: key after each move and whether that move was irreversible
  std::vector<PosKey> keys;
  std::vector<uint8_t> irreversible;

  Board() { reset(); }
  void reset() {
    pawns = BB_RANK_2 | BB_RANK_7;
    knights = bit(1) | bit(6) | bit(57) | bit(62);
    bishops = bit(2) | bit(5) | bit(58) | bit(61);
    rooks = bit(0) | bit(7) | bit(56) | bit(63);
    queens = bit(3) | bit(59);
    kings = bit(4) | bit(60);
    occ_co[WHITE] = BB_RANK_1 | BB_RANK_2;
    occ_co[BLACK] = BB_RANK_7 | BB_RANK_8;
    occ = occ_co[0] | occ_co[1];
    castling = bit(0) | bit(7) | bit(56) | bit(63);
    turn = WHITE;
    ep_square = -1;
    halfmove_clock = 0;
    fullmove = 1;
    ply = 0;
    keys.clear();
    irreversible.clear();
  }

  int piece_type_at(int sq) const {
    BB b = bit(sq);
    if (!(occ & b)) return NONE;
    if (pawns & b) return PAWN;
    if (knights & b) return KNIGHT;
    if (bishops & b) return BISHOP;
    if (rooks & b) return ROOK;
    if (queens & b) return QUEEN;
    return KING;
  }
  int king_sq(int color) const {
    BB k = kings & occ_co[color];
    return k ? msb(k) : -1;
  }
  BB attacks_from(int sq) const {
    BB b = bit(sq);
    if (pawns & b) return T().pawn_att[(occ_co[WHITE] & b) ? WHITE : BLACK][sq];
    if (knights & b) return T().knight[sq];
    if (kings & b) return T().king[sq];
    BB a = 0;
    if ((bishops | queens) & b) a |= bishop_att(sq, occ);
    if ((rooks | queens) & b) a |= rook_att(sq, occ);
    return a;
  }
  BB attackers_mask(int color, int sq, BB occupied) const {
    BB att = (T().king[sq] & kings) | (T().knight[sq] & knights) |
             (rook_att(sq, occupied) & (rooks | queens)) | (bishop_att(sq, occupied) & (bishops | queens)) |
             (T().pawn_att[color ^ 1][sq] & pawns);
    return att & occ_co[color];
  }
  BB attackers_mask(int color, int sq) const { return attackers_mask(color, sq, occ); }
  bool is_check() const {
    int k = king_sq(turn);
    return k >= 0 && attackers_mask(turn ^ 1, k) != 0;
  }

  // castling rights that are still physically possible (python-chess clean_castling_rights)
  BB clean_castling() const {
    BB c = castling & rooks;
    BB w = c & BB_RANK_1 & occ_co[WHITE], b = c & BB_RANK_8 & occ_co[BLACK];
    w &= bit(0) | bit(7);
    b &= bit(56) | bit(63);
    if (!(occ_co[WHITE] & kings & bit(4))) w = 0;
    if (!(occ_co[BLACK] & kings & bit(60))) b = 0;
    return w | b;
  }

  // ------------------------------------------------------------------ move generation
  BB slider_blockers(int king) const {
    BB rq = rooks | queens, bq = bishops | queens;
    BB snipers = ((rook_att(king, 0) & rq) | (bishop_att(king, 0) & bq)) & occ_co[turn ^ 1];
    BB blockers = 0;
    while (snipers) {
      int s = msb(snipers);
      snipers &= ~bit(s);
      BB b = T().between[king][s] & occ;
      if (b && !(b & (b - 1))) blockers |= b;
    }
    return blockers & occ_co[turn];
  }

  template <class F>
  void gen_castling(BB from_mask, BB to_mask, F&& emit) const {
    BB backrank = turn == WHITE ? BB_RANK_1 : BB_RANK_8;
    BB king = occ_co[turn] & kings & backrank & from_mask;
    if (!king) return;
    int ks = msb(king);
    BB cands = clean_castling() & backrank & to_mask;
    while (cands) {
      int rook = msb(cands);
      cands &= ~bit(rook);
      bool a_side = rook < ks;
      int king_to = (turn == WHITE ? 0 : 56) + (a_side ? 2 : 6);
      int rook_to = (turn == WHITE ? 0 : 56) + (a_side ? 3 : 5);
      BB king_path = T().between[ks][king_to], rook_path = T().between[rook][rook_to];
      if ((occ ^ king ^ bit(rook)) & (king_path | rook_path | bit(king_to) | bit(rook_to))) continue;
      BB check_sq = king_path | king;
      bool attacked = false;
      BB tmp = check_sq;
      while (tmp) {
        int s = lsb(tmp);
        tmp &= tmp - 1;
        if (attackers_mask(turn ^ 1, s, occ ^ king)) { attacked = true; break; }
      }
      if (attacked) continue;
      if (attackers_mask(turn ^ 1, king_to, occ ^ king ^ bit(rook) ^ bit(rook_to))) continue;
      emit(Move{uint8_t(ks), uint8_t(king_to), 0});
    }
  }

  template <class F>
  void gen_ep(BB from_mask, BB to_mask, F&& emit) const {
    if (ep_square < 0 || !(bit(ep_square) & to_mask)) return;
    if (bit(ep_square) & occ) return;
    BB capturers = pawns & occ_co[turn] & from_mask & T().pawn_att[turn ^ 1][ep_square] &
                   (turn == WHITE ? BB_RANK_5 : BB_RANK_4);
    while (capturers) {
      int c = msb(capturers);
      capturers &= ~bit(c);
      emit(Move{uint8_t(c), uint8_t(ep_square), 0});
    }
  }

  template <class F>
  void gen_pseudo(BB from_mask, BB to_mask, F&& emit) const {
    BB ours = occ_co[turn];
    BB non_pawns = ours & ~pawns & from_mask;
    while (non_pawns) {
      int from = msb(non_pawns);
      non_pawns &= ~bit(from);
      BB moves = attacks_from(from) & ~ours & to_mask;
      while (moves) {
        int to = msb(moves);
        moves &= ~bit(to);
        emit(Move{uint8_t(from), uint8_t(to), 0});
      }
    }
    if (from_mask & kings) gen_castling(from_mask, to_mask, emit);
    BB my_pawns = pawns & ours & from_mask;
    if (!my_pawns) return;
    BB capturers = my_pawns;
    while (capturers) {
      int from = msb(capturers);
      capturers &= ~bit(from);
      BB targets = T().pawn_att[turn][from] & occ_co[turn ^ 1] & to_mask;
      while (targets) {
        int to = msb(targets);
        targets &= ~bit(to);
        if (rank_of(to) == 0 || rank_of(to) == 7) {
          for (int p : {QUEEN, ROOK, BISHOP, KNIGHT}) emit(Move{uint8_t(from), uint8_t(to), uint8_t(p)});
        } else {
          emit(Move{uint8_t(from), uint8_t(to), 0});
        }
      }
    }
    BB single, dbl;
    if (turn == WHITE) {
      single = (my_pawns << 8) & ~occ;
      dbl = (single << 8) & ~occ & (BB_RANK_3 | BB_RANK_4);
    } else {
      single = (my_pawns >> 8) & ~occ;
      dbl = (single >> 8) & ~occ & (BB_RANK_6 | BB_RANK_5);
    }
    single &= to_mask;
    dbl &= to_mask;
    while (single) {
      int to = msb(single);
      single &= ~bit(to);
      int from = to + (turn == BLACK ? 8 : -8);
      if (rank_of(to) == 0 || rank_of(to) == 7) {
        for (int p : {QUEEN, ROOK, BISHOP, KNIGHT}) emit(Move{uint8_t(from), uint8_t(to), uint8_t(p)});
      } else {
        emit(Move{uint8_t(from), uint8_t(to), 0});
      }
    }
    while (dbl) {
      int to = msb(dbl);
      dbl &= ~bit(to);
      int from = to + (turn == BLACK ? 16 : -16);
      emit(Move{uint8_t(from), uint8_t(to), 0});
    }
    if (ep_square >= 0) gen_ep(from_mask, to_mask, emit);
  }

  bool is_en_passant(const Move& m) const {
    int diff = int(m.to) - int(m.from);
    if (diff < 0) diff = -diff;
    return ep_square == m.to && (pawns & bit(m.from)) && (diff == 7 || diff == 9) && !(occ & bit(m.to));
  }
  bool ep_skewered(int king, int capturer) const {
    int last_double = ep_square + (turn == WHITE ? -8 : 8);
    BB occupancy = (occ & ~bit(last_double) & ~bit(capturer)) | bit(ep_square);
    BB horizontal = occ_co[turn ^ 1] & (rooks | queens);
    if (rook_att(king, occupancy) & BB(0xFFull << (8 * rank_of(king))) & horizontal) return true;
    BB diagonal = occ_co[turn ^ 1] & (bishops | queens);
    if (bishop_att(king, occupancy) & diagonal) return true;
    return false;
  }
  bool is_safe(int king, BB blockers, const Move& m) const {
    if (m.from == king) {
      if (is_castling(m)) return true;
      return !attackers_mask(turn ^ 1, m.to, occ);   // python-chess: attackers with the king still on the board
    }
    if (is_en_passant(m))
      return (T().pawn_att[turn][m.from] & bit(m.to)) == bit(m.to) ? // always true for generated ep
                 ((!(blockers & bit(m.from)) || (T().ray[m.from][m.to] & bit(king))) && !ep_skewered(king, m.from))
                 : false;
    return !(blockers & bit(m.from)) || (T().ray[m.from][m.to] & bit(king));
  }
  bool is_castling(const Move& m) const {
    if (!(kings & bit(m.from))) return false;
    int diff = file_of(m.from) - file_of(m.to);
    return diff > 1 || diff < -1;
  }

  template <class F>
  void gen_evasions(int king, BB checkers, F&& emit) const {
    BB sliders = checkers & (bishops | rooks | queens);
    BB attacked = 0;
    BB tmp = sliders;
    while (tmp) {
      int c = msb(tmp);
      tmp &= ~bit(c);
      attacked |= T().ray[king][c] & ~bit(c);
    }
    BB kmoves = T().king[king] & ~occ_co[turn] & ~attacked;
    while (kmoves) {
      int to = msb(kmoves);
      kmoves &= ~bit(to);
      emit(Move{uint8_t(king), uint8_t(to), 0});
    }
    int checker = msb(checkers);
    if (bit(checker) == checkers) {
      BB target = T().between[king][checker] | checkers;
      gen_pseudo(~kings, target, emit);
      if (ep_square >= 0 && !(bit(ep_square) & target)) {
        int last_double = ep_square + (turn == WHITE ? -8 : 8);
        if (last_double == checker) gen_ep(~BB(0), ~BB(0), emit);
      }
    }
  }

  void legal_moves(std::vector<Move>& out) const {
    out.clear();
    int king = king_sq(turn);
    if (king < 0) {
      gen_pseudo(~BB(0), ~BB(0), [&](const Move& m) { out.push_back(m); });
      return;
    }
    BB blockers = slider_blockers(king);
    BB checkers = attackers_mask(turn ^ 1, king);
    auto emit = [&](const Move& m) {
      if (is_safe(king, blockers, m)) out.push_back(m);
    };
    if (checkers) gen_evasions(king, checkers, emit);
    else gen_pseudo(~BB(0), ~BB(0), emit);
  }
  bool has_legal_move() const {
    std::vector<Move> mv;
    legal_moves(mv);
    return !mv.empty();
  }
  bool has_legal_en_passant() const {
    if (ep_square < 0) return false;
    int king = king_sq(turn);
    BB blockers = king >= 0 ? slider_blockers(king) : 0;
    bool found = false;
    gen_ep(~BB(0), ~BB(0), [&](const Move& m) {
      if (king < 0 || is_safe(king, blockers, m)) {
        // an ep capture must also not leave the king in a remaining check
        Board c = light_copy();
        c.apply(m);
        int k2 = c.king_sq(turn);
        if (k2 < 0 || !c.attackers_mask(turn ^ 1, k2)) found = true;
      }
    });
    return found;
  }
  Board light_copy() const {
    Board c;
    c.pawns = pawns; c.knights = knights; c.bishops = bishops; c.rooks = rooks; c.queens = queens;
    c.kings = kings; c.occ_co[0] = occ_co[0]; c.occ_co[1] = occ_co[1]; c.occ = occ;
    c.castling = castling; c.turn = turn; c.ep_square = ep_square; c.halfmove_clock = halfmove_clock;
    c.fullmove = fullmove; c.ply = ply;
    return c;
  }

  // ------------------------------------------------------------------ make move
  bool reduces_castling_rights(const Move& m) const {
    BB cr = clean_castling();
    BB touched = bit(m.from) | bit(m.to);
    if (cr & touched) return true;
    if ((cr & BB_RANK_1) && (touched & kings & occ_co[WHITE])) return true;
    if ((cr & BB_RANK_8) && (touched & kings & occ_co[BLACK])) return true;
    return false;
  }
  bool is_zeroing(const Move& m) const {
    return (bit(m.from) & pawns) || (bit(m.to) & occ_co[turn ^ 1]) || is_en_passant(m);
  }
  void remove_piece(int sq) {
    BB m = ~bit(sq);
    pawns &= m; knights &= m; bishops &= m; rooks &= m; queens &= m; kings &= m;
    occ_co[0] &= m; occ_co[1] &= m; occ &= m;
  }
  void set_piece(int sq, int pt, int color) {
    remove_piece(sq);
    BB b = bit(sq);
    switch (pt) {
      case PAWN: pawns |= b; break;
      case KNIGHT: knights |= b; break;
      case BISHOP: bishops |= b; break;
      case ROOK: rooks |= b; break;
      case QUEEN: queens |= b; break;
      case KING: kings |= b; break;
    }
    occ_co[color] |= b;
    occ |= b;
  }
  // plays a (pseudo-)legal move without touching the repetition history
  void apply(const Move& m) {
    const bool zeroing = is_zeroing(m);
    const bool castle = is_castling(m);
    const bool ep = is_en_passant(m);
    halfmove_clock = zeroing ? 0 : halfmove_clock + 1;
    if (turn == BLACK) ++fullmove;
    const int old_ep = ep_square;
    (void)old_ep;
    ep_square = -1;
    int pt = piece_type_at(m.from);
    BB from_bb = bit(m.from), to_bb = bit(m.to);
    // castling rights
    castling &= ~from_bb & ~to_bb;
    if (pt == KING) castling &= turn == WHITE ? ~BB_RANK_1 : ~BB_RANK_8;
    if (castle) {
      bool a_side = file_of(m.to) < file_of(m.from);
      int base = turn == WHITE ? 0 : 56;
      int rook_from = base + (a_side ? 0 : 7), rook_to = base + (a_side ? 3 : 5);
      remove_piece(m.from);
      remove_piece(rook_from);
      set_piece(m.to, KING, turn);
      set_piece(rook_to, ROOK, turn);
    } else {
      if (pt == PAWN) {
        int diff = int(m.to) - int(m.from);
        if (diff == 16 && rank_of(m.from) == 1) ep_square = m.from + 8;
        else if (diff == -16 && rank_of(m.from) == 6) ep_square = m.from - 8;
        else if (ep) remove_piece(m.to + (turn == WHITE ? -8 : 8));
      }
      remove_piece(m.from);
      set_piece(m.to, m.promo ? m.promo : pt, turn);
    }
    turn ^= 1;
    ++ply;
  }
  PosKey key() const {
    PosKey k;
    std::memset(&k, 0, sizeof(k));
    k.pawns = pawns; k.knights = knights; k.bishops = bishops; k.rooks = rooks; k.queens = queens;
    k.kings = kings; k.white = occ_co[WHITE]; k.black = occ_co[BLACK]; k.castling = clean_castling();
    k.turn = turn;
    k.ep = has_legal_en_passant() ? ep_square : -1;
    return k;
  }
  void push(const Move& m) {
    // irreversible as python-chess defines it: zeroing, castling-right reducing, or played while
    // a legal en passant capture was available
    const bool irr = is_zeroing(m) || reduces_castling_rights(m) || has_legal_en_passant();
    if (keys.empty()) { keys.push_back(key()); irreversible.push_back(1); }
    apply(m);
    keys.push_back(key());
    irreversible.push_back(irr ? 1 : 0);
  }

  // ------------------------------------------------------------------ game end
  bool has_insufficient_material(int color) const {
    BB mine = occ_co[color];
    if (mine & (pawns | rooks | queens)) return false;
    if (mine & knights)
      return popcount(mine) <= 2 && !(occ_co[color ^ 1] & ~kings & ~queens);
    if (mine & bishops) {
      bool same = !(bishops & BB_DARK) || !(bishops & BB_LIGHT);
      return same && !pawns && !knights;
    }
    return true;
  }
  bool is_insufficient_material() const { return has_insufficient_material(WHITE) && has_insufficient_material(BLACK); }
  bool is_repetition(int count) const {
    if (keys.empty()) return count <= 1;
    const PosKey& cur = keys.back();
    int n = 1;
    for (int i = int(keys.size()) - 1; i > 0;) {
      if (irreversible[i]) break;   // the move that produced position i cannot be undone
      --i;
      if (keys[i] == cur && ++n >= count) return true;
    }
    return n >= count;
  }
  // 0 = game continues, 1 = checkmate, 2 = stalemate, 3 = insufficient material,
  // 4 = seventy-five moves, 5 = fivefold repetition
  int termination() const {
    bool any = has_legal_move();
    if (!any) return is_check() ? 1 : 2;
    if (is_insufficient_material()) return 3;
    if (halfmove_clock >= 150) return 4;
    if (is_repetition(5)) return 5;
    return 0;
  }
  bool is_game_over() const { return termination() != 0; }
  // -1 = no winner (draw or not over), else WHITE/BLACK
  int winner() const { return termination() == 1 ? (turn ^ 1) : -1; }
};

// ------------------------------------------------------------------ UCI text
inline std::string move_uci(const Move& m) {
  std::string s;
  s += char('a' + file_of(m.from));
  s += char('1' + rank_of(m.from));
  s += char('a' + file_of(m.to));
  s += char('1' + rank_of(m.to));
  if (m.promo) s += " pnbrqk"[m.promo];
  return s;
}
inline bool parse_uci(const char* s, Move& m) {
  size_t n = std::strlen(s);
  if (n < 4 || n > 5) return false;
  if (s[0] < 'a' || s[0] > 'h' || s[2] < 'a' || s[2] > 'h' || s[1] < '1' || s[1] > '8' || s[3] < '1' || s[3] > '8')
    return false;
  m.from = uint8_t((s[1] - '1') * 8 + (s[0] - 'a'));
  m.to = uint8_t((s[3] - '1') * 8 + (s[2] - 'a'));
  m.promo = 0;
  if (n == 5) {
    switch (s[4]) {
      case 'q': m.promo = QUEEN; break;
      case 'r': m.promo = ROOK; break;
      case 'b': m.promo = BISHOP; break;
      case 'n': m.promo = KNIGHT; break;
      default: return false;
    }
  }
  return true;
}

// Token ids of the 1968-move vocabulary: index in the generated table (same rule as
// allie_b200/moves.py).  id_of[from][to][promo-slot], promo-slot 0 = none, 1..4 = q,r,b,n.
struct MoveVocab {
  int16_t id_of[64][64][5];
  Move moves[1968];
  int n = 0;
  MoveVocab() {
    std::memset(id_of, 0xFF, sizeof(id_of));
    auto sq = [](int f, int r) { return r * 8 + f; };
    std::vector<Move> sliding, knight;
    for (int f = 0; f < 8; ++f)
      for (int r = 0; r < 8; ++r)
        for (int tr = 7; tr >= 0; --tr)
          for (int tf = 7; tf >= 0; --tf) {
            int df = tf > f ? tf - f : f - tf, dr = tr > r ? tr - r : r - tr;
            if (!df && !dr) continue;
            Move m{uint8_t(sq(f, r)), uint8_t(sq(tf, tr)), 0};
            if (df == 0 || dr == 0 || df == dr) sliding.push_back(m);
            else if ((df == 1 && dr == 2) || (df == 2 && dr == 1)) knight.push_back(m);
          }
    auto add = [&](const Move& m) {
      int slot = m.promo == 0 ? 0 : (m.promo == QUEEN ? 1 : m.promo == ROOK ? 2 : m.promo == BISHOP ? 3 : 4);
      id_of[m.from][m.to][slot] = int16_t(n);
      moves[n++] = m;
    };
    for (auto& m : sliding) add(m);
    for (auto& m : knight) add(m);
    for (int f = 0; f < 8; ++f)
      for (int side = 0; side < 2; ++side) {
        int rf = side == 0 ? 6 : 1, rt = side == 0 ? 7 : 0;
        for (int tf : {f + 1, f - 1, f}) {
          if (tf < 0 || tf > 7) continue;
          for (int p : {QUEEN, ROOK, BISHOP, KNIGHT}) add(Move{uint8_t(sq(f, rf)), uint8_t(sq(tf, rt)), uint8_t(p)});
        }
      }
  }
  int id(const Move& m) const {
    int slot = m.promo == 0 ? 0 : (m.promo == QUEEN ? 1 : m.promo == ROOK ? 2 : m.promo == BISHOP ? 3 : 4);
    return id_of[m.from][m.to][slot];
  }
};
inline const MoveVocab& vocab() {
  static const MoveVocab v;
  return v;
}

}  // namespace chess
