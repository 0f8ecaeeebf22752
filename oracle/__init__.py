"""CPU oracle for the array hot path - TEST INFRASTRUCTURE, never a product code path.

PARITY UNPINNED: the reference ships no golden vectors for this path (every check in its
tests is "compute on a Julia Array and compare"), and neither Julia nor the reference can run
in this environment.  The oracle therefore restates the SPECIFICATION the reference's tests
rely on - Julia Base semantics on `Array` - and is pinned only by closed-form known answers
(tests/golden).  Only tests, the smoke check and the benchmark's CPU baseline may import it.
"""
from .base_oracle import (broadcast, mapreduce, mapreducedim, accumulate, sort, sortperm, promote,
                          isless_key)

__all__ = ["broadcast", "mapreduce", "mapreducedim", "accumulate", "sort", "sortperm", "promote", "isless_key"]
