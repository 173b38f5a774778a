"""Stand-in OCR engines for tests: an image has no text in it, so these read a fixed word."""

CALLS = []


def reads_amber(frame) -> str:
    CALLS.append(tuple(frame.shape))
    return "amber"
