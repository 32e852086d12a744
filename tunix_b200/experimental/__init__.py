"""Distributed control plane: workers with a lifecycle state machine, remote execution, an
orchestrator with health monitoring, a transport-neutral weight-sync protocol, the RL program
loop over those pieces, a rollout service and a trajectory store."""
