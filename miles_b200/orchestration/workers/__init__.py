"""Worker management for multi-process deployments: providers of worker cells (launched here, fixed addresses, or
self-registered), a level-triggered reconcile loop, the manager that owns pools → cells → workers, and a process
supervisor.  The SPMD default (one `torchrun` rank per GPU, engines in-process) needs none of this; the HTTP engine
fleet (`--rollout-engine http --worker-provider …`) is built on it."""
