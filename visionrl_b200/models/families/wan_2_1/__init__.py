"""wan_2_1 model family."""
