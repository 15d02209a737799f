"""Assertions over a JSONL metrics file written by the trainers (`metrics_file=…`).

  python end_to_end/gpu/eval_assert.py final_loss metrics.txt 0.15 [num_samples]
  python end_to_end/gpu/eval_assert.py avg_step_time metrics.txt 0.5 [num_samples]
  python end_to_end/gpu/eval_assert.py avg_tflops metrics.txt 600 [num_samples]

Each check averages the last `num_samples` (default 10) values of its metric
(reference: end_to_end/tpu/eval_assert.py).
"""
import json
import sys

KEYS = {"final_loss": "learning/loss", "avg_step_time": "perf/step_time_seconds", "avg_tflops": "perf/per_device_tflops_per_sec"}


def last_values(path: str, key: str, n: int = 10) -> list:
  with open(path, encoding="utf8") as f:
    lines = [l for l in f if l.strip()]
  out = []
  for line in reversed(lines):
    row = json.loads(line)
    if key in row:
      out.append(float(row[key]))
      if len(out) >= n:
        break
  return out


def check(kind: str, path: str, bound: float, n: int = 10) -> float:
  if kind not in KEYS:
    raise ValueError(f"unknown check {kind}: one of {sorted(KEYS)}")
  vals = last_values(path, KEYS[kind], n)
  if not vals:
    raise ValueError(f"metric {KEYS[kind]!r} has no data points in {path}")
  mean = sum(vals) / len(vals)
  print(f"mean of the last {len(vals)} values of {KEYS[kind]}: {mean:.6g} (bound {bound:g})")
  ok = mean > bound if kind == "avg_tflops" else mean < bound
  if not ok:
    raise AssertionError(f"{kind}: {mean:.6g} is not {'above' if kind == 'avg_tflops' else 'below'} {bound:g}")
  print(f"{kind} test passed.")
  return mean


def main(argv) -> None:
  if len(argv) < 4:
    raise SystemExit(__doc__)
  check(argv[1], argv[2], float(argv[3]), int(argv[4]) if len(argv) > 4 else 10)


if __name__ == "__main__":
  main(sys.argv)
