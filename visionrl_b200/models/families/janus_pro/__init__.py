"""janus_pro model family."""
