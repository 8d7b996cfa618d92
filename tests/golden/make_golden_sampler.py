"""Makes tests/golden/ref_sample_row.json: what the reference's own samplers (``Sampler::sample``,
include/nanovllm/sampler.hpp:10-34, and the nucleus sampler ``sample_row``, sampler.hpp:46-88, compiled
unchanged with g++) pick for small random rows of logits.

    python tests/golden/make_golden_sampler.py /path/to/reference

A small driver (written here, into a temporary folder) includes the reference's header, seeds a ``std::mt19937``,
notes the number in [0, 1) that the sampler is about to draw from it (by drawing it from a copy first), calls
``sample_row`` and prints that number and the chosen token; the file records both per row.
tests/test_plain_vs_reference.py makes the same rows again (``rows`` below) and feeds them, with the recorded
numbers, to ``plain_model.sample_row``.  Rows hold no equal scores: the reference's ``std::sort``
leaves their order open.
"""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

DRIVER = r"""
#define private public            // the first sampler keeps its generator private: the driver seeds it
#include "nanovllm/sampler.hpp"
#undef private
#include <cstdio>
#include <vector>
int main() {
  int cases, first;
  if (std::scanf("%d %d", &cases, &first) != 2) return 1;
  for (int c = 0; c < first; ++c) {     // Sampler::sample (sampler.hpp:10-34): V, temperature, seed, logits
    int V;
    unsigned seed;
    double temp;
    if (std::scanf("%d %lf %u", &V, &temp, &seed) != 3) return 1;
    std::vector<float> logits(V);
    for (float& l : logits) if (std::scanf("%f", &l) != 1) return 1;
    Sampler s;
    s.rng_.seed(seed);
    std::mt19937 peek(seed);
    const double u = std::uniform_real_distribution<double>(0.0, 1.0)(peek);
    std::printf("%.17g %d\n", u, s.sample(logits.data(), V, temp));
  }
  for (int c = 0; c < cases; ++c) {
    int V, window, n_recent;
    unsigned seed;
    double temp, top_p, pen;
    if (std::scanf("%d %lf %lf %lf %d %u %d", &V, &temp, &top_p, &pen, &window, &seed, &n_recent) != 7) return 1;
    std::vector<int> recent(n_recent);
    for (int& r : recent) if (std::scanf("%d", &r) != 1) return 1;
    std::vector<float> logits(V);
    for (float& l : logits) if (std::scanf("%f", &l) != 1) return 1;
    std::mt19937 rng(seed), peek(seed);
    const double u = std::uniform_real_distribution<double>(0, 1)(peek);
    const int tok = sample_row(logits.data(), V, temp, top_p, rng, recent.data(), recent.size(), pen, window);
    std::printf("%.17g %d\n", u, tok);
  }
  return 0;
}
"""

# (temperature, top_p, penalty, window, recent ids)
PARAMS = [(0.0, 0.9, 1.0, 64, []), (1.0, 0.9, 1.0, 64, []), (0.7, 0.5, 1.0, 64, []), (1.5, 0.95, 1.0, 64, []),
          (1.0, 1.0, 1.0, 64, []), (1.0, 0.05, 1.0, 64, []), (0.8, 0.9, 1.3, 64, [3, 9, 3, 70, -1, 12]),
          (1.0, 0.8, 2.0, 2, [1, 2, 3, 4, 5]), (1.0, 0.8, 2.0, 0, [1, 2, 3, 4, 5]), (0.6, 0.7, 0.5, 64, [7, 8]),
          (1.2, 0.6, 1e20, 64, list(range(20))), (0.9, 0.0, 1.0, 64, [])]


def rows():
    """The rows of logits and their parameters (numpy's frozen RandomState stream): (logits, temperature, top_p,
    penalty, window, recent ids, seed of the reference's generator)."""
    rs = np.random.RandomState(77)
    out = []
    for rep in range(3):
        for k, (temp, top_p, pen, window, recent) in enumerate(PARAMS):
            V = (40, 64, 257)[rep]
            logits = (rs.standard_normal(V) * (1.0, 3.0, 0.3)[rep]).astype(np.float32)
            out.append((logits, temp, top_p, pen, window, recent, 1000 * rep + k))
    return out


def first_rows():
    """Rows for the engine's first sampler (``Sampler::sample``): (logits, temperature, seed)."""
    rs = np.random.RandomState(78)
    out = []
    for k, temp in enumerate((0.0, 0.3, 0.8, 1.0, 1.7, 0.01, 5.0, 0.6)):
        V = (33, 200)[k % 2]
        out.append(((rs.standard_normal(V) * 2.0).astype(np.float32), temp, 500 + k))
    return out


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden_sampler.py /path/to/reference  (a checkout of Maxritz/Nano_vLLM_cpp)")
    ref = sys.argv[1]
    work = tempfile.mkdtemp()
    with open(os.path.join(work, "driver.cpp"), "w") as f:
        f.write(DRIVER)
    exe = os.path.join(work, "driver")
    subprocess.check_call(["g++", "-std=c++20", "-O2", f"-I{ref}/include", os.path.join(work, "driver.cpp"), "-o", exe])
    cases, first = rows(), first_rows()
    text = [f"{len(cases)} {len(first)}"]
    for logits, temp, seed in first:
        text.append(f"{len(logits)} {temp!r} {seed}")
        text.append(" ".join(f"{float(x)!r}" for x in logits))
    for logits, temp, top_p, pen, window, recent, seed in cases:
        text.append(f"{len(logits)} {temp!r} {top_p!r} {pen!r} {window} {seed} {len(recent)} " + " ".join(map(str, recent)))
        text.append(" ".join(f"{float(x)!r}" for x in logits))
    out = subprocess.run([exe], input="\n".join(text) + "\n", capture_output=True, text=True, check=True).stdout.split()
    assert len(out) == 2 * (len(cases) + len(first))
    pairs = [dict(u=float(out[2 * i]), token=int(out[2 * i + 1])) for i in range(len(cases) + len(first))]
    result = dict(sample=pairs[:len(first)], sample_row=pairs[len(first):])
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_sample_row.json"), "w") as f:
        json.dump(result, f)
    print(len(first), "+", len(cases), "cases written")


if __name__ == "__main__":
    main()
