"""Multi-GPU runtime for one NVSwitch node: symmetric memory, peer-memory collectives, the sharded-parameter
engine, expert parallelism and context parallelism."""
