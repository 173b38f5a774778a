"""nextstep_1 model family."""
