// Fused extension ops (filled in below).
