"""Translation between the two config dialects of the LTX-Video transformer: the diffusers one (`LTXVideoTransformer3DModel`)
and the original `Transformer3DModel` one that this package's `LTXVideoConfig` follows
(reference: src/maxdiffusion/models/ltx_video/utils/diffusers_config_mapping.py)."""
from __future__ import annotations

_NATIVE_DEFAULTS = dict(activation_fn="gelu-approximate", attention_bias=True, attention_type="default", double_self_attention=False,
                        dropout=0.0, norm_elementwise_affine=False, norm_eps=1e-6, norm_num_groups=32, num_embeds_ada_norm=1000,
                        num_vector_embeds=None, only_cross_attention=False, upcast_attention=False, use_linear_projection=False,
                        adaptive_norm="single_scale_shift", standardization_norm="rms_norm", positional_embedding_type="rope",
                        positional_embedding_theta=10000.0, positional_embedding_max_pos=[20, 2048, 2048], timestep_scale_multiplier=1000,
                        qk_norm="rms_norm", use_tpu_flash_attention=False, sample_size=16, patch_size=1)


def diffusers_to_native(d: dict) -> dict:
  if d.get("_class_name") not in (None, "LTXVideoTransformer3DModel"):
    raise ValueError(f"not a diffusers LTX-Video transformer config: {d.get('_class_name')}")
  out = dict(_NATIVE_DEFAULTS)
  out.update(_class_name="Transformer3DModel", in_channels=d.get("in_channels", 128), out_channels=d.get("out_channels", 128),
             num_attention_heads=d.get("num_attention_heads", 32), attention_head_dim=d.get("attention_head_dim", 64),
             num_layers=d.get("num_layers", 28), cross_attention_dim=d.get("cross_attention_dim", 2048),
             caption_channels=d.get("caption_channels", 4096), norm_eps=d.get("norm_eps", 1e-6),
             norm_elementwise_affine=d.get("norm_elementwise_affine", False), attention_bias=d.get("attention_bias", True),
             qk_norm={"rms_norm_across_heads": "rms_norm"}.get(d.get("qk_norm", "rms_norm_across_heads"), d.get("qk_norm")))
  return out


def native_to_diffusers(d: dict) -> dict:
  return {"_class_name": "LTXVideoTransformer3DModel", "in_channels": d["in_channels"], "out_channels": d["out_channels"],
          "patch_size": 1, "patch_size_t": 1, "num_attention_heads": d["num_attention_heads"], "attention_head_dim": d["attention_head_dim"],
          "cross_attention_dim": d["cross_attention_dim"], "num_layers": d["num_layers"], "activation_fn": "gelu-approximate",
          "qk_norm": "rms_norm_across_heads", "norm_elementwise_affine": d.get("norm_elementwise_affine", False),
          "norm_eps": d.get("norm_eps", 1e-6), "caption_channels": d["caption_channels"], "attention_bias": d.get("attention_bias", True),
          "attention_out_bias": True}
