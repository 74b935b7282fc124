// Minimal ANSI terminal layer for the orchestui executable: raw-mode input, a cell canvas with boxes,
// text and braille line charts, flushed with escape sequences. No curses, no GUI dependency.
#pragma once
#include <poll.h>
#include <sys/ioctl.h>
#include <termios.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

namespace tui {

enum Key { KEY_NONE = 0, KEY_ENTER = 1000, KEY_ESC, KEY_UP, KEY_DOWN, KEY_LEFT, KEY_RIGHT, KEY_BACKSPACE, KEY_TAB };

enum Color { DEFAULT = 0, RED = 31, GREEN = 32, YELLOW = 33, BLUE = 34, MAGENTA = 35, CYAN = 36, GREY = 90 };

struct Cell {
  std::string glyph = " ";  // one UTF-8 code point
  int color = DEFAULT;
  bool bold = false;
};

class Canvas {
 public:
  Canvas(int w, int h) : w_(std::max(w, 20)), h_(std::max(h, 8)), cells_((size_t)w_ * h_) {}
  int width() const { return w_; }
  int height() const { return h_; }
  void clear() { std::fill(cells_.begin(), cells_.end(), Cell{}); }

  void put(int x, int y, const std::string& glyph, int color = DEFAULT, bool bold = false) {
    if (x < 0 || y < 0 || x >= w_ || y >= h_) return;
    cells_[(size_t)y * w_ + x] = Cell{glyph, color, bold};
  }
  // UTF-8 aware: one cell per code point; clipped at `max_w` cells.
  void text(int x, int y, const std::string& s, int color = DEFAULT, bool bold = false, int max_w = 1 << 20) {
    int col = 0;
    for (size_t i = 0; i < s.size() && col < max_w;) {
      const unsigned char c = (unsigned char)s[i];
      const size_t n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : 4;
      put(x + col, y, s.substr(i, n), color, bold);
      i += n;
      ++col;
    }
  }
  void box(int x, int y, int w, int h, const std::string& title = "", int color = GREY) {
    if (w < 2 || h < 2) return;
    for (int i = 1; i < w - 1; ++i) { put(x + i, y, "─", color); put(x + i, y + h - 1, "─", color); }
    for (int j = 1; j < h - 1; ++j) { put(x, y + j, "│", color); put(x + w - 1, y + j, "│", color); }
    put(x, y, "┌", color); put(x + w - 1, y, "┐", color);
    put(x, y + h - 1, "└", color); put(x + w - 1, y + h - 1, "┘", color);
    if (!title.empty()) text(x + 2, y, " " + title + " ", CYAN, true, w - 4);
  }
  // Line chart of `ys` in the cell rectangle using braille dots (2x4 sub-cells per cell).
  void chart(int x, int y, int w, int h, const std::vector<double>& ys, int color) {
    if (w < 1 || h < 1 || ys.empty()) return;
    double lo = ys[0], hi = ys[0];
    for (double v : ys) if (std::isfinite(v)) { lo = std::min(lo, v); hi = std::max(hi, v); }
    if (hi - lo < 1e-12) { hi = lo + 1e-12; }
    const int pw = w * 2, ph = h * 4;
    std::vector<uint8_t> bits((size_t)w * h, 0);
    auto plot = [&](int px, int py) {
      if (px < 0 || py < 0 || px >= pw || py >= ph) return;
      static const uint8_t dot[4][2] = {{0x01, 0x08}, {0x02, 0x10}, {0x04, 0x20}, {0x40, 0x80}};
      bits[(size_t)(py / 4) * w + px / 2] |= dot[py % 4][px % 2];
    };
    int prev_py = -1;
    for (int px = 0; px < pw; ++px) {
      const double pos = ys.size() == 1 ? 0.0 : (double)px * (double)(ys.size() - 1) / (double)std::max(1, pw - 1);
      const size_t i = std::min((size_t)pos, ys.size() - 1), i1 = std::min(i + 1, ys.size() - 1);
      const double v = ys[i] + (ys[i1] - ys[i]) * (pos - (double)i);
      if (!std::isfinite(v)) continue;
      const int py = (int)std::llround((1.0 - (v - lo) / (hi - lo)) * (ph - 1));
      if (prev_py >= 0) for (int q = std::min(prev_py, py); q <= std::max(prev_py, py); ++q) plot(px, q);
      else plot(px, py);
      prev_py = py;
    }
    for (int j = 0; j < h; ++j)
      for (int i = 0; i < w; ++i) {
        const uint8_t b = bits[(size_t)j * w + i];
        if (!b) continue;
        const uint32_t cp = 0x2800 + b;
        std::string g;
        g += (char)(0xE0 | (cp >> 12));
        g += (char)(0x80 | ((cp >> 6) & 0x3F));
        g += (char)(0x80 | (cp & 0x3F));
        put(x + i, y + j, g, color);
      }
  }
  void bar(int x, int y, int w, double frac, int color) {
    frac = std::min(1.0, std::max(0.0, frac));
    const int full = (int)std::floor(frac * w);
    for (int i = 0; i < w; ++i) put(x + i, y, i < full ? "█" : "░", i < full ? color : GREY);
  }

  // Plain rows (no escapes): used by the tests and for logs.
  std::string plain() const {
    std::string out;
    for (int j = 0; j < h_; ++j) {
      std::string row;
      for (int i = 0; i < w_; ++i) row += cells_[(size_t)j * w_ + i].glyph;
      while (!row.empty() && row.back() == ' ') row.pop_back();
      out += row + "\n";
    }
    return out;
  }
  // Full repaint with colours, cursor homed.
  std::string ansi() const {
    std::string out = "\x1b[H";
    int cur_color = -1;
    bool cur_bold = false;
    for (int j = 0; j < h_; ++j) {
      for (int i = 0; i < w_; ++i) {
        const Cell& c = cells_[(size_t)j * w_ + i];
        if (c.color != cur_color || c.bold != cur_bold) {
          out += "\x1b[0";
          if (c.bold) out += ";1";
          if (c.color) out += ";" + std::to_string(c.color);
          out += "m";
          cur_color = c.color;
          cur_bold = c.bold;
        }
        out += c.glyph;
      }
      if (j + 1 < h_) out += "\r\n";
    }
    out += "\x1b[0m";
    return out;
  }

 private:
  int w_, h_;
  std::vector<Cell> cells_;
};

// Where the UI reads keys and sends frames: a real terminal, or a script of keys (tests, demos).
class Console {
 public:
  virtual ~Console() = default;
  virtual bool usable() const = 0;
  virtual void size(int& w, int& h) const = 0;
  virtual void write(const std::string& frame) = 0;
  virtual int read_key(int timeout_ms) = 0;
  // A script may ask for the current frame to be printed (plain text) or wait for the run to finish.
  virtual bool wants_dump() { return false; }
  virtual bool waiting_for_finish() const { return false; }
  virtual void finished_now() {}
};

// Keys from a string: printable characters as themselves, and the tokens <enter> <esc> <up> <down> <left> <right> <tab>
// <bs> <wait> (hold further keys until the running session has finished) <dump> (print the frame drawn after the
// previous key). Frames are not written anywhere else; the script ends with an implicit quit.
class ScriptConsole final : public Console {
 public:
  ScriptConsole(const std::string& script, int w, int h) : w_(w), h_(h) {
    for (size_t i = 0; i < script.size();) {
      if (script[i] == '<') {
        const size_t e = script.find('>', i);
        const std::string tok = e == std::string::npos ? "" : script.substr(i + 1, e - i - 1);
        int k = -1;
        if (tok == "enter") k = KEY_ENTER; else if (tok == "esc") k = KEY_ESC; else if (tok == "up") k = KEY_UP;
        else if (tok == "down") k = KEY_DOWN; else if (tok == "left") k = KEY_LEFT; else if (tok == "right") k = KEY_RIGHT;
        else if (tok == "tab") k = KEY_TAB; else if (tok == "bs") k = KEY_BACKSPACE; else if (tok == "wait") k = -2; else if (tok == "dump") k = -3;
        if (k != -1) { keys_.push_back(k); i = e + 1; continue; }
      }
      keys_.push_back((unsigned char)script[i++]);
    }
  }
  bool usable() const override { return true; }
  void size(int& w, int& h) const override { w = w_; h = h_; }
  void write(const std::string&) override {}
  int read_key(int timeout_ms) override {
    if (waiting_) { ::usleep((useconds_t)std::min(timeout_ms, 50) * 1000); return KEY_NONE; }
    while (pos_ < keys_.size()) {
      const int k = keys_[pos_++];
      if (k == -2) { waiting_ = true; return KEY_NONE; }
      if (k == -3) { dump_ = true; return KEY_NONE; }
      return k;
    }
    return exhausted_++ < 3 ? KEY_NONE : 'Q';     // a few more frames, then the hard quit key
  }
  bool wants_dump() override { const bool d = dump_; dump_ = false; return d; }
  bool waiting_for_finish() const override { return waiting_; }
  void finished_now() override { waiting_ = false; }

 private:
  int w_, h_;
  std::vector<int> keys_;
  size_t pos_ = 0;
  int exhausted_ = 0;
  bool waiting_ = false, dump_ = false;
};

class Terminal final : public Console {
 public:
  Terminal() {
    tty_ = ::isatty(STDIN_FILENO) && ::isatty(STDOUT_FILENO);
    if (!tty_) return;
    ::tcgetattr(STDIN_FILENO, &saved_);
    termios raw = saved_;
    raw.c_lflag &= ~(ECHO | ICANON | ISIG | IEXTEN);
    raw.c_iflag &= ~(IXON | ICRNL);
    raw.c_cc[VMIN] = 0;
    raw.c_cc[VTIME] = 0;
    ::tcsetattr(STDIN_FILENO, TCSAFLUSH, &raw);
    write("\x1b[?1049h\x1b[?25l");  // alternate screen, hide cursor
  }
  ~Terminal() {
    if (!tty_) return;
    write("\x1b[?25h\x1b[?1049l");
    ::tcsetattr(STDIN_FILENO, TCSAFLUSH, &saved_);
  }
  bool is_tty() const { return tty_; }
  bool usable() const override { return tty_; }
  void size(int& w, int& h) const override {
    winsize ws{};
    if (tty_ && ::ioctl(STDOUT_FILENO, TIOCGWINSZ, &ws) == 0 && ws.ws_col > 0) { w = ws.ws_col; h = ws.ws_row; }
    else { w = 100; h = 32; }
  }
  void write(const std::string& s) override {
    size_t off = 0;
    while (off < s.size()) {
      ssize_t k = ::write(STDOUT_FILENO, s.data() + off, s.size() - off);
      if (k <= 0) break;
      off += (size_t)k;
    }
  }
  // Next key (printable ASCII as itself) or KEY_NONE after `timeout_ms`.
  int read_key(int timeout_ms) override {
    pollfd pf{STDIN_FILENO, POLLIN, 0};
    if (::poll(&pf, 1, timeout_ms) <= 0) return KEY_NONE;
    unsigned char c;
    if (::read(STDIN_FILENO, &c, 1) != 1) return KEY_NONE;
    if (c == '\r' || c == '\n') return KEY_ENTER;
    if (c == 127 || c == 8) return KEY_BACKSPACE;
    if (c == '\t') return KEY_TAB;
    if (c == 3) return 'q';  // ctrl-c behaves like quit
    if (c != 27) return c;
    pollfd p2{STDIN_FILENO, POLLIN, 0};
    if (::poll(&p2, 1, 20) <= 0) return KEY_ESC;
    unsigned char seq[2] = {0, 0};
    if (::read(STDIN_FILENO, &seq[0], 1) != 1 || seq[0] != '[') return KEY_ESC;
    if (::read(STDIN_FILENO, &seq[1], 1) != 1) return KEY_ESC;
    switch (seq[1]) {
      case 'A': return KEY_UP;
      case 'B': return KEY_DOWN;
      case 'C': return KEY_RIGHT;
      case 'D': return KEY_LEFT;
    }
    return KEY_NONE;
  }

 private:
  bool tty_ = false;
  termios saved_{};
};

}  // namespace tui
