"""Offline dataset preparation: pre-encoded latents + text embeddings -> sharded TFRecord files."""
