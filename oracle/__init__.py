"""CPU checker for the TurboQuant hot path.  Test infrastructure only: the shipped package never
imports anything from this folder."""
