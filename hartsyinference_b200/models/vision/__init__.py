"""Vision models beyond the embedders: super-resolution, depth."""
