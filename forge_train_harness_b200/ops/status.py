"""Codes of the device status word (``csrc/common.cuh::StatusCode``): which bounded wait of an sm_100a kernel gave up."""

STATUS_NAMES = {1: "shared-memory stage never filled", 2: "shared-memory stage never released",
                3: "accumulator never committed", 4: "accumulator never drained", 5: "peer flag never set", 6: "timeout",
                7: "an input index lies outside its valid range (debug input check)"}
