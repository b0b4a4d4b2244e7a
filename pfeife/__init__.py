"""Import-path compatibility: ``pfeife.option``, ``pfeife.mp``, ``pfeife.mp.partial``,
``pfeife.loss``, ``pfeife.batch``, ``pfeife.utils``, ``pfeife.timing``, ``pfeife.compile``,
``pfeife.device_bench``, ``pfeife.graph.*``, ``pfeife.schedule.*``, ``pfeife.local.*`` resolve
to the implementations in ``pfeife_b200`` so that a script written against the reference runs
unchanged."""
