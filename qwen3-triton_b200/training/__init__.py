"""Host side of the training loop's data path and validation (import path of the reference's top-level `training`
package): token blocks from a flat uint32 corpus and exact full-coverage validation."""
