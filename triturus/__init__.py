"""Drop-in import paths of the reference package: `triturus.lm2exp`, `triturus.lt2exp`, `triturus.utils`
resolve to the sm_100a implementation in `triturus_b200`, so code written against the reference
(`from triturus.lm2exp import lm2exp`) runs unchanged."""
