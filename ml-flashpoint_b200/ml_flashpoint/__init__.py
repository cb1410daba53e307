"""ML Flashpoint checkpoint save / restore / replication data path, B200-native.

The package keeps the module paths of the reference project (``ml_flashpoint.core``,
``ml_flashpoint.checkpoint_object_manager``, ``ml_flashpoint.replication``,
``ml_flashpoint.adapter``) so that it can stand in for it. Bytes are moved by the CUDA kernels
behind ``libmlf_b200.so``; see ``ml_flashpoint._native``.
"""
