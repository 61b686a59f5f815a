"""Launch accounting: every op wrapper that launches one of this library's kernels bumps a counter, so that a
benchmark can report how many of the library's own kernels ran inside its timed region (replays of a captured
graph count the launches recorded at capture time)."""
LAUNCHES = 0


def bump(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


def get() -> int:
    return LAUNCHES
