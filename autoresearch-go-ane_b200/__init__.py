"""B200-native drop-in for the training-step hot path of tmc/autoresearch-go-ane.

The product is `lib/libane_b200.so` (C ABI, see include/ane_b200.h).  `ane/` is a thin
Python mirror of the reference's Go `ane` package used by the tests and the benchmark;
`go/ane/` holds the purego binding for Go hosts.
"""
