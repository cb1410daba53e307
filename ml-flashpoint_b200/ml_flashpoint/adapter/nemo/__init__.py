"""NeMo 2.0 / Lightning integration of the B200 checkpoint data path (needs nemo, lightning, megatron-core)."""
