"""Self-contained recipes on synthetic cached latents: no checkpoints, datasets or codec needed."""
