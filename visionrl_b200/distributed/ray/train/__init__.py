"""Train actors."""
