"""Channels-last execution of the Wan 2.1 VAE decoder on the implicit-GEMM convolution kernels.

`AutoencoderKLWan.decode` hands CUDA bf16 latents to `ChannelsLastDecoder`, which walks the same modules (and therefore
the same parameters) as the NCDHW PyTorch path but keeps every activation as `[B, T, H, W, C]`:

  * 3x3x3 causal convolutions and the (3,1,1) time convolution run on `ops.conv.conv3d_causal`; the 2-frame feature
    cache of a convolution is the history tensor the kernel reads its negative-time taps from, so nothing is
    concatenated in front of a chunk (reference: src/maxdiffusion/models/wan/autoencoder_kl_wan.py:70-147);
  * `RMS_norm -> SiLU` is one row kernel; bias and the residual add ride in the convolution's epilogue (:452-484);
  * nearest-2x + 3x3 conv is the fused low-resolution form (`ops.conv.upsample2x_conv2d`), and the time up-sampling
    writes its two channel halves straight into the even / odd frames of the output (:245-389) -- no interleave pass;
  * 1x1 convolutions are GEMMs on the tcgen05 GEMM kernel.

The mid-block attention (one head of 384 channels over the H*W positions of a frame, :487-546) is two GEMMs around a
row-softmax kernel (`ops.conv.wide_head_attention`): the flash kernels of this repository are built for head sizes
64 and 128, and a latent frame has few enough positions for the score matrix to be materialised.

Spatial parallelism (`decode(.., spatial=HaloExchange)`): every rank decodes a vertical strip of the frame. The input
of a 3x3 convolution is produced with one spare column on each side (`ops.conv.rms_act(halo=1)`, or a convolution
writing into the interior of a wider tensor), the neighbours' edge columns are exchanged into them
(`parallel.spatial.HaloExchange.fill`) and the convolution reads them without producing output for them. The 2-frame
histories keep their halos, so a later chunk exchanges only its own frames. The mid-block attention gathers the
latent frame (a few thousand positions) and every rank keeps its strip of the result.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from ...ops import conv as OC
from ...ops import kernels as K


class _Hist:
  """The last two input frames of every cached convolution, by call order within a pass (channels-last)."""

  def __init__(self):
    self.slots: list = []
    self.cursor = 0

  def begin_pass(self):
    self.cursor = 0

  def next(self) -> int:
    i = self.cursor
    self.cursor += 1
    if i >= len(self.slots):
      self.slots.append(None)
    return i


def _roll_history(hist: Optional[torch.Tensor], x: torch.Tensor) -> torch.Tensor:
  """The two frames that precede the NEXT chunk: the tail of [hist | x] (zeros where the clip has not started)."""
  if x.shape[1] >= 2:
    return x[:, -2:]
  prev = hist[:, 1:] if hist is not None else torch.zeros_like(x)
  return torch.cat([prev, x], dim=1)


class ChannelsLastDecoder:

  def __init__(self, vae):
    self.vae = vae
    self._packed: dict = {}
    self.halo = None  # `parallel.spatial.HaloExchange` while a width-sharded decode runs

  # ---- packed weights (re-packed when a parameter changes) -----------------------------------
  def _pack(self, key, params, make):
    ver = tuple((p.data_ptr(), p._version) for p in params if p is not None)
    hit = self._packed.get(key)
    if hit is None or hit[0] != ver:
      hit = (ver, make())
      self._packed[key] = hit
    return hit[1]

  def _conv3_pack(self, m):
    return self._pack(id(m), (m.weight, m.bias), lambda: OC.pack_conv3d(m.weight.detach(), None if m.bias is None else m.bias.detach()))

  # ---- layers ----------------------------------------------------------------------------------
  def conv3(self, m, x, hist: Optional[_Hist], residual=None, haloed: bool = False):
    """A `WanCausalConv3d`: x [B, T, H, W, Ci] -> [B, T, H, W, Co]. Width-sharded: `haloed` says that x already has
    its two spare columns (still to be filled from the neighbours); otherwise x is copied into a wider tensor."""
    kt = m.weight.shape[2]
    if tuple(m.weight.shape[2:]) == (1, 1, 1):
      return self.pointwise(m.weight, m.bias, x, residual)
    pk = self._conv3_pack(m)
    x = OC.pad_channels(x, pk.c_in)
    spatial = self.halo is not None and m.weight.shape[-1] > 1
    if spatial:
      x = self.halo.fill(x) if haloed else self.halo.extend(x)
    past = None
    if hist is not None and kt > 1:
      slot = hist.next()
      past = hist.slots[slot]
      hist.slots[slot] = _roll_history(past, x)  # with its halo columns: later chunks exchange only their own frames
    return OC.conv3d_causal(x, pk, hist=past, residual=residual, halo=1 if spatial else 0)

  def pointwise(self, weight, bias, x, residual=None):
    """1x1(x1) convolution = GEMM over the pixel rows."""
    co, ci = weight.shape[:2]
    w2 = self._pack(("pw", id(weight)), (weight, bias),
                    lambda: (weight.detach().reshape(co, ci).to(torch.bfloat16).contiguous(),
                             None if bias is None else bias.detach().to(torch.bfloat16).contiguous()))
    rows = x.reshape(-1, ci)
    if not OC.use_kernel(x):
      y = F.linear(rows, weight.reshape(co, ci).to(x.dtype), None if bias is None else bias.to(x.dtype))
      if residual is not None:
        y = y + residual.reshape(-1, co)
    elif ci % 64 or co % 8:
      y = F.linear(rows, w2[0], w2[1])
      if residual is not None:
        y = y + residual.reshape(-1, co)
    elif residual is not None:
      y = K.gemm(rows, w2[0], bias=w2[1], epi="add_res", residual=residual.reshape(-1, co))
    else:
      y = K.gemm(rows, w2[0], bias=w2[1])
    return y.reshape(*x.shape[:-1], co)

  def norm(self, m, x, silu: bool, for_conv: bool = False):
    """`for_conv`: the result feeds a 3x3 convolution; width-sharded it gets the two spare columns for the halo."""
    return OC.rms_act(x.contiguous(), m.gamma, m.bias, silu=silu, halo=1 if (for_conv and self.halo is not None) else 0)

  def res_block(self, blk, x, hist):
    h = self.conv3(blk.conv_shortcut, x, None) if blk.conv_shortcut is not None else x
    y = self.conv3(blk.conv1, self.norm(blk.norm1, x, True, for_conv=True), hist, haloed=True)
    return self.conv3(blk.conv2, self.norm(blk.norm2, y, True, for_conv=True), hist, residual=h.contiguous(), haloed=True)

  def attention(self, blk, x):
    if self.halo is not None:
      # every position attends to the whole frame: gather the strips (latent resolution), keep this rank's columns
      return self.halo.shard(self._attention(blk, self.halo.gather(x.contiguous())))
    return self._attention(blk, x)

  def _attention(self, blk, x):
    B, T, H, W, C = x.shape
    y = self.norm(blk.norm, x, False)
    qkv = self.pointwise(blk.to_qkv.weight, blk.to_qkv.bias, y).reshape(B * T, H * W, 3, C)
    # one head of C channels over the H * W positions of every frame: GEMM -> row softmax -> GEMM on this
    # repository's kernels (the flash kernels are built for head sizes 64 and 128)
    o = torch.stack([OC.wide_head_attention(qkv[f, :, 0], qkv[f, :, 1], qkv[f, :, 2]) for f in range(B * T)])
    return self.pointwise(blk.proj.weight, blk.proj.bias, o.reshape(B, T, H, W, C), residual=x.contiguous())

  def resample(self, rs, x, hist, first_chunk: bool):
    B, T, H, W, C = x.shape
    if rs.mode == "upsample3d":
      if hist is None:
        if T > 1:  # whole clip: the first frame stays single, every later frame is doubled
          x = torch.cat([x[:, :1], self._time_upsample(rs, x[:, 1:], None)], dim=1)
      elif first_chunk:
        hist.next()  # the first frame skips the time convolution but keeps the slot order of later chunks
      else:
        x = self._time_upsample(rs, x, hist)
    T2 = x.shape[1]
    conv = rs.resample[1]
    pk = self._pack(("up", id(conv)), (conv.weight, conv.bias), lambda: OC.pack_upsample_conv2d(conv.weight.detach(), conv.bias.detach()))
    x = x.reshape(B * T2, H, W, C)
    if self.halo is not None:
      x = self.halo.extend(x)
    y = OC.upsample2x_conv2d(x, pk, halo=0 if self.halo is None else 1)
    return y.reshape(B, T2, 2 * H, 2 * W, y.shape[-1])

  def _time_upsample(self, rs, x, hist: Optional[_Hist]):
    """(3,1,1) causal conv C -> 2C whose channel halves become the even / odd output frames."""
    m = rs.time_conv
    B, T, H, W, C = x.shape
    halves = self._pack(("tc", id(m)), (m.weight, m.bias),
                        lambda: [OC.pack_conv3d(m.weight.detach()[j * C:(j + 1) * C], m.bias.detach()[j * C:(j + 1) * C]) for j in range(2)])
    past = None
    if hist is not None:
      slot = hist.next()
      past = hist.slots[slot]
      hist.slots[slot] = _roll_history(past, x)
    out = torch.empty((B, 2 * T, H, W, C), dtype=x.dtype, device=x.device)
    for j in range(2):
      OC.conv3d_causal(x, halves[j], hist=past, out=out[:, j::2])
    return out

  @staticmethod
  def dup_up(sc, x, first_chunk: bool):
    """`WanDupUp3D` of the 2.2 VAE, channels-last: every input channel is repeated, and the repeated channels are
    dealt out over a (time factor, 2, 2) block of output positions -- a parameter-free shortcut around an up block
    (reference: src/maxdiffusion/models/wan/autoencoder_kl_wan.py, `DupUp3D`). x [B, T, H, W, C] ->
    [B, T ft, 2H, 2W, cout]; the first chunk drops the frames in front of its only real one."""
    B, T, H, W, C = x.shape
    ft, fs, co = sc.ft, sc.fs, sc.cout
    idx = torch.arange(co * ft * fs * fs, device=x.device) // sc.repeats
    y = x[..., idx].reshape(B, T, H, W, co, ft, fs, fs).permute(0, 1, 5, 2, 6, 3, 7, 4)  # B, T, ft, H, fs, W, fs, co
    y = y.reshape(B, T * ft, H * fs, W * fs, co)
    return y[:, ft - 1:] if first_chunk else y

  # ---- decoder ---------------------------------------------------------------------------------
  def decoder(self, x, hist: Optional[_Hist], first_chunk: bool):
    from .autoencoder_kl_wan import WanResample

    d = self.vae.decoder
    x = self.conv3(d.conv_in, x, hist)
    mid = d.mid_block
    x = self.res_block(mid.resnets[0], x, hist)
    x = self.attention(mid.attentions[0], x)
    x = self.res_block(mid.resnets[1], x, hist)
    for up in d.up_blocks:
      if hasattr(up, "avg_shortcut"):
        # Wan 2.2: residual blocks and the resampler in one list, plus a parameter-free shortcut around the block
        h = x
        for layer in up.resnets:
          h = self.resample(layer, h, hist, first_chunk) if isinstance(layer, WanResample) else self.res_block(layer, h, hist)
        x = h + self.dup_up(up.avg_shortcut, x, first_chunk or hist is None) if up.avg_shortcut is not None else h
        continue
      for r in up.resnets:
        x = self.res_block(r, x, hist)
      if up.upsamplers is not None:
        x = self.resample(up.upsamplers[0], x, hist, first_chunk)
    return self.conv3(d.conv_out, self.norm(d.norm_out, x, True, for_conv=True), hist, haloed=True)

  # ---- encoder ---------------------------------------------------------------------------------
  def downsample(self, rs, x, state: dict, chunked: bool, first_chunk: bool):
    """`WanResample` in a down mode: 3x3 stride-2 convolution with the padding on the far side (`ZeroPad2d((0,1,0,1))`),
    then for `downsample3d` the (3,1,1) time convolution with stride 2 over [last frame of the previous chunk | this
    chunk] (reference: src/maxdiffusion/models/wan/autoencoder_kl_wan.py:245-389). The strided time convolution is the
    causal one evaluated at every second frame: output j reads frames (2j-1, 2j, 2j+1) of the chunk, frame -1 being
    the remembered one."""
    B, T, H, W, C = x.shape
    conv = rs.resample[1]
    pk = self._pack(("down", id(conv)), (conv.weight, conv.bias),
                    lambda: OC.pack_conv2d(conv.weight.detach(), conv.bias.detach(), stride=2, pad_top_left=0))
    y = OC.conv2d(x.reshape(B * T, H, W, C), pk)
    y = y.reshape(B, T, H // 2, W // 2, y.shape[-1])
    if rs.mode != "downsample3d":
      return y
    m = rs.time_conv
    tk = self._pack(("tdown", id(m)), (m.weight, m.bias), lambda: OC.pack_conv3d(m.weight.detach(), m.bias.detach()))
    if chunked and first_chunk:
      state[id(rs)] = y[:, -1:].clone()
      return y
    if chunked:
      last, body = state[id(rs)], y
      state[id(rs)] = y[:, -1:].clone()
    else:
      if T == 1:
        return y
      last, body = y[:, :1], y[:, 1:]
    out = OC.conv3d_causal(body.contiguous(), tk, hist=torch.cat([last, last], dim=1).contiguous())[:, 1::2]
    return out if chunked else torch.cat([y[:, :1], out], dim=1)

  def encoder(self, x, hist: Optional[_Hist], state: dict, first_chunk: bool):
    from .autoencoder_kl_wan import WanResample, WanResidualBlock

    e = self.vae.encoder
    x = self.conv3(e.conv_in, x, hist)
    for blk in e.down_blocks:
      if isinstance(blk, WanResample):
        x = self.downsample(blk, x, state, hist is not None, first_chunk)
      elif isinstance(blk, WanResidualBlock):
        x = self.res_block(blk, x, hist)
      else:
        x = self.attention(blk, x)
    mid = e.mid_block
    x = self.res_block(mid.resnets[0], x, hist)
    x = self.attention(mid.attentions[0], x)
    x = self.res_block(mid.resnets[1], x, hist)
    return self.conv3(e.conv_out, self.norm(e.norm_out, x, True), hist)

  @torch.no_grad()
  def encode(self, x: torch.Tensor, chunk: int = 4, whole_clip: bool = False) -> torch.Tensor:
    """x [B, 3, T, H, W] in [-1, 1] (T = 1 + 4k) -> the moments [B, 2 z, T', H / 8, W / 8] that `DiagonalGaussian`
    takes: the encoder on the convolution kernels, frames in chunks of `chunk` after the first one."""
    vae = self.vae
    x = x.permute(0, 2, 3, 4, 1).contiguous()
    state: dict = {}
    if whole_clip:
      h = self.encoder(x, None, state, True)
    else:
      hist = _Hist()
      outs, start, first, t = [], 0, True, x.shape[1]
      while start < t:
        n = 1 if first else min(chunk, t - start)
        hist.begin_pass()
        outs.append(self.encoder(x[:, start:start + n], hist, state, first))
        start += n
        first = False
      h = torch.cat(outs, dim=1)
    h = self.pointwise(vae.quant_conv.weight, vae.quant_conv.bias, h.contiguous())
    return h.permute(0, 4, 1, 2, 3)

  @torch.no_grad()
  def decode(self, z: torch.Tensor, chunk: int = 1, whole_clip: bool = False, spatial=None) -> torch.Tensor:
    """z [B, 16, T', H', W'] (de-normalised latents, bf16, CUDA) -> video [B, 3, 1 + 4 (T' - 1), 8 H', 8 W'] in [-1, 1].
    `spatial` (`parallel.spatial.HaloExchange`): z is replicated over its group, every rank decodes the strip
    [rank W'/n, (rank + 1) W'/n) of the latent width and all ranks return the whole video."""
    if spatial is not None and spatial.size > 1 and z.shape[-1] % spatial.size == 0:
      self.halo = spatial
      # the largest edge column of the decode: frames x rows x channels peaks at 4 * 8 * 96 = 4 * 4 * 192 per latent
      # frame and row (time x 4, height x 8 at 96 channels); 4096 leaves room for the channel padding
      frames = z.shape[2] if whole_clip else max(1, chunk)
      spatial.reserve(4096 * z.shape[0] * frames * z.shape[3], z.dtype)
      try:
        strip = self._decode(spatial.shard(z, dim=-1), chunk, whole_clip)
      finally:
        self.halo = None
      return spatial.gather(strip.contiguous(), dim=-1)
    return self._decode(z, chunk, whole_clip)

  def _decode(self, z, chunk, whole_clip):
    vae = self.vae
    x = z.permute(0, 2, 3, 4, 1).contiguous()  # channels-last
    x = self.pointwise(vae.post_quant_conv.weight, vae.post_quant_conv.bias, x)
    if whole_clip:
      out = self.decoder(x, None, True)
    else:
      hist = _Hist()
      outs, start, first, t = [], 0, True, x.shape[1]
      while start < t:
        n = 1 if first else min(chunk, t - start)
        hist.begin_pass()
        outs.append(self.decoder(x[:, start:start + n], hist, first))
        start += n
        first = False
      out = torch.cat(outs, dim=1)
    p = int(getattr(vae.cfg, "patch_size", 1))
    if p > 1:
      # Wan 2.2 folds a p x p pixel patch into the channels: channel c p^2 + r p + q is pixel (q, r) of the patch
      B, T, H, W, _ = out.shape
      out = out[..., :3 * p * p].reshape(B, T, H, W, 3, p, p).permute(0, 1, 2, 6, 3, 5, 4).reshape(B, T, H * p, W * p, 3)
    return out.clamp_(-1.0, 1.0).permute(0, 4, 1, 2, 3)
