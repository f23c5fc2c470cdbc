//! `PolyOps` (`prover/poly/circle/ops.rs:16-145`). The library keeps its own twiddle tower per context (every canonic
//! domain's twiddles are slices of it), so `Twiddles` carries nothing and `precompute_twiddles` only records the coset:
//! the precondition `domain.half_coset.is_doubling_of(twiddles.root_coset)` is checked as the other backends check it.
use std::ffi::c_void;

use itertools::Itertools;
use stwo::core::circle::{CirclePoint, Coset};
use stwo::core::fields::m31::BaseField;
use stwo::core::fields::qm31::SecureField;
use stwo::core::poly::circle::{CanonicCoset, CircleDomain};
use stwo::core::ColumnVec;
use stwo::prover::air::component_prover::Poly;
use stwo::prover::backend::{Col, Column};
use stwo::prover::poly::circle::{CircleCoefficients, CircleEvaluation, PolyOps};
use stwo::prover::poly::twiddles::TwiddleTree;
use stwo::prover::poly::BitReversedOrder;

use crate::column::{B200BaseColumn, B200SecureColumn, DeviceWords};
use crate::ctx::{check, ctx, B200Backend};
use crate::ffi;

fn point_words(p: CirclePoint<SecureField>) -> [u32; 8] {
    let (x, y) = (p.x.to_m31_array(), p.y.to_m31_array());
    [x[0].0, x[1].0, x[2].0, x[3].0, y[0].0, y[1].0, y[2].0, y[3].0]
}
fn secure(w: [u32; 4]) -> SecureField { SecureField::from_u32_unchecked(w[0], w[1], w[2], w[3]) }

impl PolyOps for B200Backend {
    type Twiddles = ();

    fn interpolate(eval: CircleEvaluation<Self, BaseField, BitReversedOrder>, twiddles: &TwiddleTree<Self>) -> CircleCoefficients<Self> {
        Self::interpolate_columns(vec![eval], twiddles).pop().unwrap()
    }

    // One launch sequence per size group, in place in the columns it was given (they are consumed).
    fn interpolate_columns(columns: Vec<CircleEvaluation<Self, BaseField, BitReversedOrder>>, twiddles: &TwiddleTree<Self>) -> Vec<CircleCoefficients<Self>> {
        let mut by_log: std::collections::BTreeMap<u32, Vec<*mut u32>> = Default::default();
        for c in &columns {
            assert!(c.domain.half_coset.is_doubling_of(twiddles.root_coset));
            by_log.entry(c.domain.log_size()).or_default().push(c.values.0.ptr);
        }
        for (log, ptrs) in by_log {
            check(unsafe { ffi::zkb_ifft_cols(ctx(), ptrs.as_ptr(), ptrs.len() as i32, log as i32) });
        }
        columns.into_iter().map(|c| CircleCoefficients::new(c.values)).collect()
    }

    fn eval_at_point(poly: &CircleCoefficients<Self>, point: CirclePoint<SecureField>) -> SecureField {
        Self::batch_eval_at_point(&[poly], point)[0]
    }

    fn batch_eval_at_point(polys: &[&CircleCoefficients<Self>], point: CirclePoint<SecureField>) -> Vec<SecureField> {
        if polys.is_empty() {
            return Vec::new();
        }
        let log = polys[0].log_size();
        assert!(polys.iter().all(|p| p.log_size() == log));
        let ptrs = polys.iter().map(|p| p.coeffs.0.ptr as *const u32).collect_vec();
        let mut out = vec![0u32; 4 * ptrs.len()];
        check(unsafe { ffi::zkb_eval_at_point_cols(ctx(), ptrs.as_ptr(), ptrs.len() as i32, log as i32, point_words(point).as_ptr(), out.as_mut_ptr()) });
        out.chunks_exact(4).map(|w| secure([w[0], w[1], w[2], w[3]])).collect()
    }

    fn barycentric_weights(coset: CanonicCoset, p: CirclePoint<SecureField>) -> Col<Self, SecureField> {
        let w = DeviceWords::uninit(4 << coset.log_size());
        check(unsafe { ffi::zkb_barycentric_weights(ctx(), coset.log_size() as i32, point_words(p).as_ptr(), w.ptr) });
        B200SecureColumn(w)
    }

    fn barycentric_eval_at_point(evals: &CircleEvaluation<Self, BaseField, BitReversedOrder>, weights: &Col<Self, SecureField>) -> SecureField {
        let mut out = [0u32; 4];
        check(unsafe { ffi::zkb_barycentric_eval_at_point(ctx(), evals.values.0.ptr, weights.0.ptr, evals.domain.log_size() as i32, out.as_mut_ptr()) });
        secure(out)
    }

    fn eval_at_point_by_folding(evals: &CircleEvaluation<Self, BaseField, BitReversedOrder>, point: CirclePoint<SecureField>, _twiddles: &TwiddleTree<Self>) -> SecureField {
        let mut out = [0u32; 4];
        check(unsafe { ffi::zkb_eval_at_point_by_folding(ctx(), evals.values.0.ptr, evals.domain.log_size() as i32, point_words(point).as_ptr(), out.as_mut_ptr()) });
        secure(out)
    }

    fn extend(poly: &CircleCoefficients<Self>, log_size: u32) -> CircleCoefficients<Self> {
        assert!(log_size >= poly.log_size());
        let out = DeviceWords::zeros(1 << log_size);
        check(unsafe { ffi::zkb_d2d(ctx(), out.ptr as *mut c_void, poly.coeffs.0.ptr as *const c_void, poly.coeffs.len() * 4) });
        CircleCoefficients::new(B200BaseColumn(out))
    }

    fn evaluate(poly: &CircleCoefficients<Self>, domain: CircleDomain, twiddles: &TwiddleTree<Self>) -> CircleEvaluation<Self, BaseField, BitReversedOrder> {
        assert!(domain.half_coset.is_doubling_of(twiddles.root_coset));
        // The extension is implicit: the transform reads coeffs[idx mod n] where the layers above the coefficient count
        // would only copy (no zero-extended copy of the polynomial is made).
        let out = DeviceWords::uninit(domain.size());
        let (src, dst) = ([poly.coeffs.0.ptr as *const u32], [out.ptr]);
        check(unsafe { ffi::zkb_lde_cols(ctx(), src.as_ptr(), 1, poly.log_size() as i32, dst.as_ptr(), domain.log_size() as i32) });
        CircleEvaluation::new(domain, B200BaseColumn(out))
    }

    fn evaluate_polynomials(polynomials: ColumnVec<CircleCoefficients<Self>>, log_blowup_factor: u32, twiddles: &TwiddleTree<Self>, store_polynomials_coefficients: bool) -> Vec<Poly<Self>> {
        // one launch sequence per coefficient size, all columns of that size together
        let outs = polynomials.iter().map(|p| DeviceWords::uninit(1 << (p.log_size() + log_blowup_factor))).collect_vec();
        let mut by_log: std::collections::BTreeMap<u32, (Vec<*const u32>, Vec<*mut u32>)> = Default::default();
        for (p, o) in polynomials.iter().zip(&outs) {
            let e = by_log.entry(p.log_size()).or_default();
            e.0.push(p.coeffs.0.ptr);
            e.1.push(o.ptr);
        }
        for (log, (src, dst)) in by_log {
            let domain = CanonicCoset::new(log + log_blowup_factor).circle_domain();
            assert!(domain.half_coset.is_doubling_of(twiddles.root_coset));
            check(unsafe { ffi::zkb_lde_cols(ctx(), src.as_ptr(), src.len() as i32, log as i32, dst.as_ptr(), (log + log_blowup_factor) as i32) });
        }
        polynomials.into_iter().zip(outs).map(|(coeffs, o)| {
            let domain = CanonicCoset::new(coeffs.log_size() + log_blowup_factor).circle_domain();
            Poly::new(store_polynomials_coefficients.then_some(coeffs), CircleEvaluation::new(domain, B200BaseColumn(o)))
        }).collect()
    }

    fn precompute_twiddles(coset: Coset) -> TwiddleTree<Self> {
        crate::ctx::init(0, coset.log_size() + 2);  // the tower covers the circle domains built on this half coset
        TwiddleTree { root_coset: coset, twiddles: (), itwiddles: () }
    }

    fn split_at_mid(poly: CircleCoefficients<Self>) -> (CircleCoefficients<Self>, CircleCoefficients<Self>) {
        let (l, r) = poly.coeffs.split_at_mid();
        (CircleCoefficients::new(l), CircleCoefficients::new(r))
    }
}
