"""Small how-to scripts: each is runnable as `python -m maxdiffusion_b200.pedagogical_examples.<name>` and shows one
part of the framework in isolation (reference: src/maxdiffusion/pedagogical_examples/)."""
