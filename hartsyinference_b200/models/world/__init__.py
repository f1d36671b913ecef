"""Interactive world models: frame-by-frame video generation conditioned on player actions."""
