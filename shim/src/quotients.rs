//! `QuotientOps` (`prover/pcs/quotient_ops.rs:19-43`).
use itertools::Itertools;
use stwo::core::constraints::complex_conjugate_line_coeffs;
use stwo::core::fields::m31::BaseField;
use stwo::core::fields::qm31::SecureField;
use stwo::core::pcs::quotients::{ColumnSampleBatch, PointSample};
use stwo::core::poly::circle::CanonicCoset;
use stwo::prover::backend::Column;
use stwo::prover::pcs::quotient_ops::{AccumulatedNumerators, QuotientOps};
use stwo::prover::poly::circle::{CircleEvaluation, SecureEvaluation};
use stwo::prover::poly::BitReversedOrder;
use num_traits::Zero;

use crate::ctx::{check, ctx, B200Backend};
use crate::ffi;
use crate::fri::{coords, coords_mut, new_secure, words};

impl QuotientOps for B200Backend {
    fn accumulate_numerators(columns: &[&CircleEvaluation<Self, BaseField, BitReversedOrder>], sample_batches: &[ColumnSampleBatch], accumulated_numerators_vec: &mut Vec<AccumulatedNumerators<Self>>) {
        let log = columns[0].domain.log_size();
        let ptrs = columns.iter().map(|c| c.values.0.ptr as *const u32).collect_vec();
        for batch in sample_batches {
            // line coefficients (core/pcs/quotients.rs:229-258); the kernel takes b and c, the `a` terms are summed here
            let (mut idx, mut b, mut c) = (Vec::new(), Vec::new(), Vec::new());
            let mut first = SecureField::zero();
            for nd in &batch.cols_vals_randpows {
                let (la, lb, lc) = complex_conjugate_line_coeffs(&PointSample { point: batch.point, value: nd.sample_value }, nd.random_coeff);
                idx.push(nd.column_index as u32);
                b.extend(words(lb));
                c.extend(words(lc));
                first += la;
            }
            let mut acc = new_secure(1 << log);
            check(unsafe { ffi::zkb_quot_numerators(ctx(), ptrs.as_ptr(), ptrs.len() as i32, log as i32, idx.as_ptr(), b.as_ptr(), c.as_ptr(), idx.len() as i32, coords_mut(&mut acc).as_ptr()) });
            accumulated_numerators_vec.push(AccumulatedNumerators { sample_point: batch.point, partial_numerators_acc: acc, first_linear_term_acc: first });
        }
    }

    fn compute_quotients_and_combine(accs: Vec<AccumulatedNumerators<Self>>, lifting_log_size: u32) -> SecureEvaluation<Self, BitReversedOrder> {
        let (mut cols, mut logs, mut first, mut pts) = (Vec::new(), Vec::new(), Vec::new(), Vec::new());
        for a in &accs {
            cols.extend(coords(&a.partial_numerators_acc));
            logs.push(a.partial_numerators_acc.len().ilog2() as i32);
            first.extend(words(a.first_linear_term_acc));
            pts.extend(words(a.sample_point.x));
            pts.extend(words(a.sample_point.y));
        }
        let mut out = new_secure(1 << lifting_log_size);
        check(unsafe { ffi::zkb_quot_combine(ctx(), accs.len() as i32, cols.as_ptr(), logs.as_ptr(), first.as_ptr(), pts.as_ptr(), lifting_log_size as i32, coords_mut(&mut out).as_ptr()) });
        SecureEvaluation::new(CanonicCoset::new(lifting_log_size).circle_domain(), out)
    }
}
