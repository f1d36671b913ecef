"""Model families: ``llm`` (decoder LLMs, MoE, MLA), ``dit`` (Flux-class image DiT, Wan-class video
DiT), ``encoders`` (T5 / CLIP text encoders), ``vae`` (2-D and causal 3-D decoders)."""
