"""Python harness shared by bench.py, the smoke check and the tests: seeded problem generators
(cases), the synthetic networks of the benchmark configurations as operator lists that both a
CPU checker and the device engine can run (mobilenet_v1, resnet50), and a writer for MACE's
model-file wire format (netdef_wire).  Nothing here is on the product path; functions that
need a CPU checker receive it as an argument."""
