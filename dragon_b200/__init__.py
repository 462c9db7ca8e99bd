"""B200-native `Collective` path of Dragon: C-ABI library, operator layer and
the distributed Python APIs.  Nothing here imports the CPU oracle."""

__version__ = "0.1.0"
