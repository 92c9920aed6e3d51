"""Parallel runtime pieces beyond plain data parallelism: the sharded optimizer, peer-memory
(NVLink) collectives, context-parallel attention and expert-parallel dispatch."""
