"""Minimum versions of the packages this framework imports. `required` ones are checked at import; the others only
when the feature that needs them is used (reference: src/maxdiffusion/dependency_versions_table.py)."""
deps = {
    "torch": "torch>=2.6",
    "numpy": "numpy>=1.26",
    "pyyaml": "pyyaml>=5.1",
    "safetensors": "safetensors>=0.4",
    "transformers": "transformers>=4.44",
    "sentencepiece": "sentencepiece>=0.1.99",
    "pillow": "pillow>=9.0",
    "datasets": "datasets>=2.14",
    "tensorboard": "tensorboard>=2.12",
    "imageio": "imageio>=2.31",
    "av": "av>=10.0",
    "ninja": "ninja>=1.10",
}
required = ("torch", "numpy", "pyyaml", "safetensors")
