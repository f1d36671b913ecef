"""Text encoders of the diffusion pipelines: T5 / umT5 (encoder only) and CLIP text."""
