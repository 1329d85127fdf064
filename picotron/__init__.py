"""Import paths of the reference package, served by ``picotron_b200``.

A script written against the reference (``from picotron.tensor_parallel.tensor_parallel import
apply_tensor_parallel``, ``import picotron.process_group_manager as pgm`` ...) imports unchanged:
every module here *is* the corresponding ``picotron_b200`` module (the same module object is
registered under both names), so module-level state such as
``picotron.process_group_manager.process_group_manager`` is shared, not copied.
"""
