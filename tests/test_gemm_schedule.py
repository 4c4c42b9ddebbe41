"""The work schedule of the persistent tensor-core GEMM (``rllama_b200/csrc/gemm_sched.h``) checked on the host: a
small C++ program built with g++ walks the schedule exactly as the kernel's three roles and its fix-up do, for model
shapes and random ones, and verifies that every (tile, k-block) unit is computed exactly once, that pieces follow k
order inside a CTA's run, that a CTA leaves at most two partial tiles, and that the fix-up finds precisely the partial
tiles the pieces wrote, in k order. No GPU needed."""
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r"""
#include <cstdio>
#include <cstdlib>
#include <map>
#include <vector>
#include "gemm_sched.h"
using namespace gemm_sched;

static int check(int n, int M, int nkb, int grid, int TN, int TT) {
    const Sched s = make_sched(n, M, nkb, grid, TN, TT);
    const int tiles = s.n_mt * s.n_nt;
    std::vector<int> covered((size_t)tiles * nkb, 0);
    // (tile -> list of (kb0, slab)) as the pieces write them
    std::map<int, std::vector<std::pair<int, int>>> written;
    for (int c = 0; c < grid; c++) {
        PieceIter it(s, c, grid);
        Piece p;
        int partials = 0, last_tile = -1;
        bool seen0 = false, seen1 = false;
        while (it.next(p)) {
            if (p.tile < 0 || p.tile >= tiles || p.kb0 < 0 || p.kb1 > nkb || p.kb0 >= p.kb1) return 1;
            for (int kb = p.kb0; kb < p.kb1; kb++) covered[(size_t)p.tile * nkb + kb]++;
            if (p.slot >= 0) {
                if (p.tile < s.whole) return 2;               // whole tiles are never partial
                partials++;
                if (p.slot == 0) { if (seen0) return 3; seen0 = true; }
                else if (p.slot == 1) { if (seen1) return 3; seen1 = true; }
                else return 3;
                written[p.tile].push_back({p.kb0, c * 2 + p.slot});
            } else if (p.kb0 != 0 || p.kb1 != nkb) return 4;   // a direct piece covers the whole K range
            if (p.tile >= s.whole && last_tile >= s.whole && p.tile < last_tile) return 5;  // tile-major runs
            last_tile = p.tile;
        }
        if (partials > 2) return 6;
    }
    for (int v : covered) if (v != 1) return 7;
    // the fix-up's view of every remaining tile
    for (int j = 0; j < s.rest; j++) {
        std::vector<int> slabs;
        for (int c = 0; c < grid; c++) {
            const int slab = partial_of(s, grid, j, c);
            if (slab >= 0) slabs.push_back(slab);
        }
        const auto it = written.find(s.whole + j);
        if (slabs.size() == 1) { if (it != written.end()) return 8; continue; }  // computed whole by one CTA
        if (it == written.end() || it->second.size() != slabs.size()) return 9;
        int prev_kb = -1;
        for (size_t i = 0; i < slabs.size(); i++) {
            if (it->second[i].second != slabs[i]) return 10;   // same partial tiles, same (CTA = k) order
            if (it->second[i].first <= prev_kb) return 11;
            prev_kb = it->second[i].first;
        }
    }
    return 0;
}

int main(int argc, char** argv) {
    // n M K grid TN TT lines on stdin
    int n, M, K, grid, TN, TT, bad = 0, cases = 0;
    while (scanf("%d %d %d %d %d %d", &n, &M, &K, &grid, &TN, &TT) == 6) {
        const int nkb = (K + 63) / 64;
        const int r = check(n, M, nkb, grid, TN, TT);
        cases++;
        if (r) { printf("FAIL %d: n %d M %d K %d grid %d TN %d TT %d\n", r, n, M, K, grid, TN, TT); bad++; }
    }
    printf("%d cases, %d bad\n", cases, bad);
    return bad ? 1 : 0;
}
"""


def test_every_unit_is_computed_once_and_the_fixup_finds_the_partials(tmp_path):
    src = tmp_path / "sched_check.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "sched_check"
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "rllama_b200", "csrc"), str(src), "-o", str(exe)])
    lines = []
    # the projections of the 7B / 13B / 30B / 65B layers (whole and per tensor-parallel rank) at the benchmark prompts
    for d, F, heads in ((4096, 11008, 32), (5120, 13824, 40), (6656, 17920, 52), (8192, 22016, 64)):
        for tp in (1, 2, 4, 8):
            nq = (heads // tp + (1 if heads % tp else 0)) * (d // heads)
            for n in (16, 64, 128, 129, 512, 1792):
                for (M, K) in ((3 * nq, d), (d, nq), (2 * F // tp, d), (d, F // tp)):
                    for grid in (148, 132):
                        units = ((n + 127) // 128) * ((M + 127) // 128) * ((K + 63) // 64)
                        lines.append("%d %d %d %d 128 128" % (n, M, K, min(grid, units)))
                        units = ((n + 127) // 128) * ((M + 255) // 256) * ((K + 63) // 64)
                        lines.append("%d %d %d %d 256 128" % (n, M, K, min(grid, units)))
                        units = ((n + 255) // 256) * ((M + 255) // 256) * ((K + 63) // 64)
                        lines.append("%d %d %d %d 256 256" % (n, M, K, min(grid, units)))
    rng = np.random.default_rng(0)
    for _ in range(3000):
        n, M, K = int(rng.integers(1, 3000)), int(rng.integers(1, 50000)), int(rng.integers(8, 30000))
        TN, TT = [(128, 128), (256, 128), (256, 256)][int(rng.integers(0, 3))]
        units = ((n + TT - 1) // TT) * ((M + TN - 1) // TN) * ((K + 63) // 64)
        grid = int(min(rng.integers(1, 257), units))
        lines.append("%d %d %d %d %d %d" % (n, M, K, grid, TN, TT))
    out = subprocess.run([str(exe)], input="\n".join(lines) + "\n", capture_output=True, text=True)
    assert out.returncode == 0, out.stdout[-2000:]
    assert "0 bad" in out.stdout
