"""cosmos model family."""
