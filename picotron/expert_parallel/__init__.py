"""``picotron.expert_parallel``: see the modules of this package (aliases of ``picotron_b200.parallel``)."""
