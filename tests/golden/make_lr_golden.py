"""Generates tests/golden/lr_schedule.json from the reference's own header-only LearningRateScheduler
(include/optim/lr_scheduler.h:9-55): a few lines of C++ that include the header from the reference checkout are compiled
with g++ and run here; nothing of the reference is copied. Usage: python tests/golden/make_lr_golden.py [<checkout>]"""
import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
CASES = [(3e-4, 3e-5, 10, 100), (3e-4, 0.0, 0, 7), (1e-3, 1e-4, 1, 2), (6e-4, 6e-5, 1177, 58874), (1e-4, 1e-4, 3, 10)]
PROGRAM = r'''
#include "optim/lr_scheduler.h"
#include <cstdio>
#include <cstdlib>
int main(int argc, char** argv) {
    const float lr = std::strtof(argv[1], nullptr), mn = std::strtof(argv[2], nullptr);
    const std::size_t warm = std::strtoull(argv[3], nullptr, 10), total = std::strtoull(argv[4], nullptr, 10);
    LearningRateScheduler s({lr, mn, warm, total});
    for (int i = 5; i < argc; ++i) std::printf("%.9g\n", s.learning_rate(std::strtoull(argv[i], nullptr, 10)));
}
'''


def main() -> None:
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("CGPT_REFERENCE", str(HERE.parent.parent.parent / "reference")))
    out = []
    with tempfile.TemporaryDirectory() as tmp:
        src, exe = Path(tmp) / "lr.cpp", Path(tmp) / "lr"
        src.write_text(PROGRAM)
        subprocess.run(["/usr/bin/g++", "-std=c++20", "-O2", "-I", str(ref / "include"), str(src), "-o", str(exe)], check=True)
        for lr, mn, warm, total in CASES:
            steps = sorted({0, 1, 2, warm - 1 if warm else 0, warm, warm + 1, total // 3, total // 2, total - 3, total - 2, total - 1, total, total + 5} - {-1, -2, -3})
            steps = [s for s in steps if s >= 0]
            res = subprocess.run([str(exe), repr(lr), repr(mn), str(warm), str(total), *map(str, steps)], check=True, capture_output=True, text=True)
            out.append({"initial": lr, "minimum": mn, "warmup": warm, "total": total, "steps": steps,
                        "values": [float(v) for v in res.stdout.split()]})
    (HERE / "lr_schedule.json").write_text(json.dumps(out, indent=1))
    print(f"wrote {HERE / 'lr_schedule.json'} ({sum(len(c['steps']) for c in out)} values)")


if __name__ == "__main__":
    main()
