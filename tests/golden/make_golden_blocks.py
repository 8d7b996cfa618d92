"""Makes tests/golden/ref_block_manager.json: the block tables that the reference's own ``BlockManager``
(src/block_manager.cpp, compiled unchanged with g++) hands out over a scripted life of a few requests with
common prefixes: admission with prefix hits, whole prompts, decoding across page edges, hashing of pages as
they fill, release, revival of freed pages that still carry a hash, and the order in which fresh pages leave
the free list.

    python tests/golden/make_golden_blocks.py /path/to/reference

The driver (written here, into a temporary folder) reads the script below and does with each request what the
reference's scheduler does (src/scheduler.cpp:27-53, 57-77, 90-108): ``can_allocate`` and ``allocate`` on
admission, ``may_append`` before a decode step, ``hash_blocks`` after a step, ``deallocate`` at the end.  After
every line it prints the request's block table and the number of free blocks.
tests/test_cache_scheduler_cpu.py replays the same script on this engine's cache manager (and on its plain
restatement) and compares page for page.  Pages hold 4 tokens here; the pool has 10.
"""
import json
import os
import subprocess
import sys
import tempfile

PAGE, PAGES = 4, 10
P = list(range(100, 108))                    # a common prefix of two full pages
# ("admit", name, tokens) | ("decode", name, token that the step appends) | ("end", name)
SCRIPT = [
    ("admit", "a", P + [1, 2, 3]),           # 11 tokens: two full pages and a part
    ("admit", "b", P + [4, 5, 6]),           # shares a's two full pages
    ("decode", "a", 7),                      # a: 12 tokens, its third page fills with the next row
    ("decode", "a", 8),                      # a: 13 tokens: a fourth page
    ("decode", "b", 9),
    ("admit", "c", P[:4] + [50, 51, 52, 53, 54]),     # shares only the first page
    ("end", "a"),                            # a's own pages go back (in reverse), the shared ones stay
    ("admit", "d", P + [1, 2, 3, 7, 60, 61]),         # revives a's freed third page by its hash
    ("end", "b"),
    ("end", "c"),
    ("admit", "e", [70, 71, 72, 73, 74, 75, 76, 77, 78]),   # fresh pages: the order of the free list shows
    ("decode", "e", 79),
    ("decode", "e", 80),
    ("decode", "e", 81),
    ("decode", "e", 82),                     # e: 13 tokens: a fourth page
    ("end", "d"),
    ("end", "e"),
    ("admit", "f", P + [1, 2, 3, 7, 60, 61, 62, 63, 64]),   # everything is free; hashed pages are revived
    ("admit", "g", P[:4] + [50, 51, 52, 53, 54, 55]),
    ("end", "g"),
    ("end", "f"),
]

DRIVER = r"""
#include "nanovllm/block_manager.hpp"
#include <cstdio>
#include <map>
#include <memory>
#include <string>
int main() {
  int page, pages, lines;
  if (std::scanf("%d %d %d", &page, &pages, &lines) != 3) return 1;
  Sequence::block_size = page;
  BlockManager m(pages, page);
  std::map<std::string, std::unique_ptr<Sequence>> live;
  SamplingParams sp;
  for (int l = 0; l < lines; ++l) {
    char op[16], name[16];
    if (std::scanf("%15s %15s", op, name) != 2) return 1;
    std::string o(op), n(name);
    int cached = -2;
    if (o == "admit") {                                   // src/scheduler.cpp:27-53 and 90-99, a whole prompt
      int len;
      if (std::scanf("%d", &len) != 1) return 1;
      std::vector<int> ids(len);
      for (int& t : ids) if (std::scanf("%d", &t) != 1) return 1;
      live[n] = std::make_unique<Sequence>(ids, sp);
      Sequence& s = *live[n];
      cached = m.can_allocate(s);
      if (cached >= 0) {
        m.allocate(s, cached);
        s.num_scheduled_tokens = s.num_tokens - s.num_cached_tokens;
        m.hash_blocks(s);
        s.num_cached_tokens += s.num_scheduled_tokens;
        s.num_scheduled_tokens = 0;
      }
    } else if (o == "decode") {                           // src/scheduler.cpp:57-77 and 90-99
      int tok;
      if (std::scanf("%d", &tok) != 1) return 1;
      Sequence& s = *live[n];
      s.append_token(tok);                                // the token the step before drew
      if (!m.can_append(s)) return 2;
      m.may_append(s);
      s.num_scheduled_tokens = 1;
      m.hash_blocks(s);
      s.num_cached_tokens += 1;
      s.num_scheduled_tokens = 0;
    } else {
      m.deallocate(*live[n]);
    }
    std::printf("%d %d", cached, m.free_count());
    for (int b : live[n]->block_table) std::printf(" %d", b);
    std::printf("\n");
    if (o == "end") live.erase(n);
  }
  return 0;
}
"""


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden_blocks.py /path/to/reference  (a checkout of Maxritz/Nano_vLLM_cpp)")
    ref = sys.argv[1]
    work = tempfile.mkdtemp()
    with open(os.path.join(work, "driver.cpp"), "w") as f:
        f.write(DRIVER)
    exe = os.path.join(work, "driver")
    subprocess.check_call(["g++", "-std=c++20", "-O2", f"-I{ref}/include", os.path.join(work, "driver.cpp"),
                           f"{ref}/src/block_manager.cpp", "-o", exe])
    text = [f"{PAGE} {PAGES} {len(SCRIPT)}"]
    for line in SCRIPT:
        if line[0] == "admit":
            text.append(f"admit {line[1]} {len(line[2])} " + " ".join(map(str, line[2])))
        elif line[0] == "decode":
            text.append(f"decode {line[1]} {line[2]}")
        else:
            text.append(f"end {line[1]}")
    out = subprocess.run([exe], input="\n".join(text) + "\n", capture_output=True, text=True, check=True).stdout
    result = []
    for row in out.strip().splitlines():
        v = [int(x) for x in row.split()]
        result.append(dict(cached_pages=v[0], free=v[1], table=v[2:]))
    assert len(result) == len(SCRIPT)
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_block_manager.json"), "w") as f:
        json.dump(result, f)
    for line, r in zip(SCRIPT, result):
        print(line[:2], r)


if __name__ == "__main__":
    main()
