"""TEST INFRASTRUCTURE ONLY.  CPU restatement of the reference's PyTorch full chain
(attention -> O_proj -> AllReduce) used as the parity checker.  Nothing in the
product package may import this; only the tests, the smoke entry and the bench's
CPU-baseline leg do."""
