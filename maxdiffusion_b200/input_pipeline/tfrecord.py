"""TFRecord / tf.train.Example / serialized-tensor reader and writer without TensorFlow.

The Wan training data of the reference are TFRecords of `tf.train.Example`s whose bytes features `latents` and
`encoder_hidden_states` hold `tf.io.serialize_tensor` output (float32), eval records add an int64 `timesteps`
(src/maxdiffusion/trainers/wan_trainer.py:84-112, input_pipeline/_tfds_data_processing.py:83-166, writer side
data_preprocessing/wan_pusav1_to_tfrecords.py:73-138). TensorFlow is not a dependency here, so the three layers are
implemented directly: the record framing (length, masked CRC32C, payload, masked CRC32C), the protobuf wire format
of Example / Features / Feature / BytesList / FloatList / Int64List, and TensorProto (dtype, shape, tensor_content).
"""
from __future__ import annotations

import struct
from typing import Dict, Iterator, List, Union

import numpy as np

# ---------------------------------------------------------------------------------------------- CRC32C
_CRC_TABLE = None


def _crc_table():
  global _CRC_TABLE
  if _CRC_TABLE is None:
    poly = 0x82F63B78
    t = np.zeros(256, dtype=np.uint32)
    for i in range(256):
      c = i
      for _ in range(8):
        c = (c >> 1) ^ poly if c & 1 else c >> 1
      t[i] = c
    _CRC_TABLE = t
  return _CRC_TABLE


def crc32c(data: bytes) -> int:
  t = _crc_table()
  c = 0xFFFFFFFF
  for b in data:
    c = int(t[(c ^ b) & 0xFF]) ^ (c >> 8)
  return c ^ 0xFFFFFFFF


def masked_crc(data: bytes) -> int:
  c = crc32c(data)
  return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


# ---------------------------------------------------------------------------------------------- framing
def read_records(path: str, verify: bool = False) -> Iterator[bytes]:
  with open(path, "rb") as f:
    while True:
      head = f.read(12)
      if len(head) < 12:
        return
      (length,), (len_crc,) = struct.unpack("<Q", head[:8]), struct.unpack("<I", head[8:])
      if verify and masked_crc(head[:8]) != len_crc:
        raise ValueError(f"{path}: corrupt record header")
      data = f.read(length)
      (data_crc,) = struct.unpack("<I", f.read(4))
      if verify and masked_crc(data) != data_crc:
        raise ValueError(f"{path}: corrupt record payload")
      yield data


def write_records(path: str, records, with_crc: bool = True) -> None:
  with open(path, "wb") as f:
    for data in records:
      head = struct.pack("<Q", len(data))
      f.write(head + struct.pack("<I", masked_crc(head) if with_crc else 0))
      f.write(data + struct.pack("<I", masked_crc(data) if with_crc else 0))


# ---------------------------------------------------------------------------------------------- protobuf wire
def _varint(buf: bytes, pos: int):
  out = shift = 0
  while True:
    b = buf[pos]
    pos += 1
    out |= (b & 0x7F) << shift
    if not b & 0x80:
      return out, pos
    shift += 7


def _enc_varint(v: int) -> bytes:
  v &= (1 << 64) - 1
  out = bytearray()
  while True:
    b = v & 0x7F
    v >>= 7
    out.append(b | (0x80 if v else 0))
    if not v:
      return bytes(out)


def _fields(buf: bytes):
  pos = 0
  while pos < len(buf):
    key, pos = _varint(buf, pos)
    num, wt = key >> 3, key & 7
    if wt == 0:
      val, pos = _varint(buf, pos)
    elif wt == 1:
      val, pos = buf[pos:pos + 8], pos + 8
    elif wt == 2:
      n, pos = _varint(buf, pos)
      val, pos = buf[pos:pos + n], pos + n
    elif wt == 5:
      val, pos = buf[pos:pos + 4], pos + 4
    else:
      raise ValueError(f"unsupported wire type {wt}")
    yield num, wt, val


def _ld(num: int, payload: bytes) -> bytes:
  return _enc_varint((num << 3) | 2) + _enc_varint(len(payload)) + payload


Feature = Union[List[bytes], np.ndarray]


def parse_example(data: bytes) -> Dict[str, Feature]:
  """tf.train.Example -> {name: list of bytes | float32 array | int64 array}."""
  out: Dict[str, Feature] = {}
  for num, _, features in _fields(data):
    if num != 1:
      continue
    for fnum, _, entry in _fields(features):
      if fnum != 1:
        continue
      name, feat = None, b""
      for enum, _, val in _fields(entry):
        if enum == 1:
          name = val.decode()
        elif enum == 2:
          feat = val
      for knum, _, lst in _fields(feat):
        if knum == 1:
          out[name] = [v for n, _, v in _fields(lst) if n == 1]
        elif knum == 2:
          vals = []
          for n, wt, v in _fields(lst):
            vals.append(np.frombuffer(v, dtype="<f4"))
          out[name] = np.concatenate(vals) if vals else np.zeros(0, np.float32)
        elif knum == 3:
          vals = []
          for n, wt, v in _fields(lst):
            if wt == 0:
              vals.append(v)
            else:
              p = 0
              while p < len(v):
                x, p = _varint(v, p)
                vals.append(x)
          out[name] = np.array([x - (1 << 64) if x >= (1 << 63) else x for x in vals], dtype=np.int64)
  return out


def make_example(features: Dict[str, Feature]) -> bytes:
  entries = b""
  for name, value in features.items():
    if isinstance(value, (list, tuple)) and (not value or isinstance(value[0], (bytes, bytearray))):
      feat = _ld(1, b"".join(_ld(1, bytes(v)) for v in value))
    else:
      arr = np.asarray(value)
      if arr.dtype.kind == "f":
        feat = _ld(2, _ld(1, arr.astype("<f4").tobytes()))
      else:
        feat = _ld(3, _ld(1, b"".join(_enc_varint(int(x)) for x in arr.reshape(-1))))
    entries += _ld(1, _ld(1, name.encode()) + _ld(2, feat))
  return _ld(1, entries)


_DT = {1: np.float32, 2: np.float64, 3: np.int32, 9: np.int64, 14: "bfloat16", 19: np.float16}
_DT_INV = {np.dtype(np.float32): 1, np.dtype(np.float64): 2, np.dtype(np.int32): 3, np.dtype(np.int64): 9, np.dtype(np.float16): 19}


def parse_tensor(data: bytes) -> np.ndarray:
  """`tf.io.parse_tensor` for dense numeric tensors stored in `tensor_content`."""
  dtype, shape, content = 1, [], b""
  for num, _, val in _fields(data):
    if num == 1:
      dtype = val
    elif num == 2:
      for n2, _, dim in _fields(val):
        if n2 == 2:
          size = 0
          for n3, _, v in _fields(dim):
            if n3 == 1:
              size = v
          shape.append(size)
    elif num == 4:
      content = val
  if _DT.get(dtype) == "bfloat16":
    raw = np.frombuffer(content, dtype="<u2").astype(np.uint32) << 16
    return raw.view(np.float32).reshape(shape)
  return np.frombuffer(content, dtype=np.dtype(_DT[dtype]).newbyteorder("<")).reshape(shape)


def serialize_tensor(arr: np.ndarray) -> bytes:
  arr = np.ascontiguousarray(arr)
  shape = b"".join(_ld(2, _enc_varint((1 << 3) | 0) + _enc_varint(int(s))) for s in arr.shape)
  return _enc_varint((1 << 3) | 0) + _enc_varint(_DT_INV[arr.dtype]) + _ld(2, shape) + _ld(4, arr.tobytes())
