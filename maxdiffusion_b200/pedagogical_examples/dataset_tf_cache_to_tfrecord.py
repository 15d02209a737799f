"""Re-shards an existing folder of TFRecord files (for instance one big cached file) into `no_records_per_shard`-sized
shards so that every data-parallel rank gets whole files.

  python -m maxdiffusion_b200.pedagogical_examples.dataset_tf_cache_to_tfrecord <src_dir> <dst_dir> <records_per_shard>
"""
from __future__ import annotations

import glob
import os
import sys

from ..data_preprocessing.tfrecord_shards import ShardedWriter
from ..input_pipeline.tfrecord import read_records


def run(src: str, dst: str, per_shard: int) -> list:
  writer = ShardedWriter(dst, per_shard)
  for f in sorted(set(glob.glob(os.path.join(src, "*.tfrec*")))):
    for rec in read_records(f, verify=True):
      writer.write(rec)
  files = writer.close()
  print(f"{writer.total} records -> {len(files)} shards under {dst}")
  return files


if __name__ == "__main__":
  run(sys.argv[1], sys.argv[2], int(sys.argv[3]))
