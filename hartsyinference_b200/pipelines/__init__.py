"""Generation pipelines: Flux (image), Wan (video)."""
