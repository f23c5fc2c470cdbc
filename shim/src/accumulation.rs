//! `AccumulationOps` (`prover/air/accumulation.rs:127-145`).
use stwo::core::fields::qm31::SecureField;
use stwo::prover::backend::Column;
use stwo::prover::secure_column::SecureColumnByCoords;
use stwo::prover::AccumulationOps;
use num_traits::One;

use crate::ctx::{check, ctx, B200Backend};
use crate::ffi;
use crate::fri::{coords, coords_mut};

impl AccumulationOps for B200Backend {
    fn accumulate(column: &mut SecureColumnByCoords<Self>, other: &SecureColumnByCoords<Self>) {
        assert_eq!(column.len(), other.len());
        check(unsafe { ffi::zkb_accumulate(ctx(), coords_mut(column).as_ptr(), coords(other).as_ptr(), column.len()) });
    }

    fn generate_secure_powers(felt: SecureField, n_powers: usize) -> Vec<SecureField> {
        // a few hundred field multiplications on the host (cpu/accumulation.rs:17-26)
        let mut out = Vec::with_capacity(n_powers);
        let mut acc = SecureField::one();
        for _ in 0..n_powers {
            out.push(acc);
            acc *= felt;
        }
        out
    }

    fn lift_and_accumulate(cols: Vec<SecureColumnByCoords<Self>>) -> Option<SecureColumnByCoords<Self>> {
        let mut it = cols.into_iter();
        let mut acc = it.next()?;
        for mut next in it {  // ascending sizes: next = next + lift(acc)
            let (ls, ld) = (acc.len().ilog2() as i32, next.len().ilog2() as i32);
            check(unsafe { ffi::zkb_lift_accumulate(ctx(), coords_mut(&mut next).as_ptr(), ld, coords(&acc).as_ptr(), ls) });
            acc = next;
        }
        Some(acc)
    }
}
