"""sd3_5 model family."""
