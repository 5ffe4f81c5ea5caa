"""CPU oracle for the paged-decode hot path. Test infrastructure only."""
