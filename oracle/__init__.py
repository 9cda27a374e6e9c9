"""Test infrastructure only: CPU restatements of the reference's W4A4 path used as the parity checker and as the
timed CPU baseline.  Nothing in the shipped package imports this directory."""
